// Building blocks shared by the library's own multi-block kernels (collectives, MoE dispatch and
// combine, fused GEMM + collective): block-paired cross-PE barriers, an intra-kernel grid barrier,
// launch helpers that understand several PEs per process.
#pragma once

#include <cuda_runtime.h>

#include "rocshmem/rocshmem.h"

namespace rocshmem {
namespace kernels {

using detail::st;

// Symmetric kernel arguments are given as addresses on the process's first local PE and are rebased
// to the block's own PE. Plain device pointers (ordinary torch tensors) are passed through, which
// is what a process with one PE per GPU uses for its private inputs and outputs.
template <typename T>
__device__ __forceinline__ T *rebase(T *p) {
  const rocshmem_device_state &s = st();
  const char *c = reinterpret_cast<const char *>(p);
  if (c >= s.window_base && c < s.window_base + size_t(s.n_pes) * s.heap_stride) return detail::local_ptr(p);
  return p;
}

// Cross-PE barrier between "the same block" on every member of a team: block b of a PE signals
// block b of every member and waits for all of them. Blocks of one PE never wait for each other, so
// a kernel built on this needs no grid-wide synchronisation and no cooperative launch when each PE
// has its own GPU. All members must launch the same number of blocks for the same sequence of
// library calls on a team, which keeps the per-(team, block) epochs in step without communication.
// Returns false if a peer did not arrive within the wait budget (error record written).
//
// `publish` == false is the cheaper "I am done reading" form: the flags are written and polled with
// relaxed accesses (no system-scope fence). It orders nothing the block wrote, so it may only be used
// where the block has no data to hand over, e.g. before a source buffer is released for reuse.
__device__ inline bool block_pair_barrier(const rocshmem_team_dev *t, unsigned block, bool publish = true) {
  __shared__ unsigned long long s_epoch;
  const rocshmem_device_state &s = st();
  const unsigned tid = detail::block_tid(), nthr = detail::block_threads();
  __syncthreads();
  if (t->size == 1) return true;  // nobody to pair with (every member skips, so epochs stay in step)
  if (tid == 0) {
    unsigned long long *e = s.lib_state + size_t(t->slot) * ROCSHMEM_LIB_MAX_BLOCKS + block;
    s_epoch = *e + 1;
    *e = s_epoch;
  }
  __syncthreads();
  const unsigned long long epoch = s_epoch;
  unsigned long long *mine =
      s.lib_flags + (size_t(t->slot) * ROCSHMEM_LIB_MAX_BLOCKS + block) * ROCSHMEM_MAX_PES;
  bool ok = true;
  if (publish) {
    for (unsigned j = tid; j < static_cast<unsigned>(t->size); j += nthr) {
      detail::st_release_sys(detail::remote_ptr(mine + t->my_pe, detail::team_pe_to_world(t, j)), epoch);
    }
    for (unsigned j = tid; j < static_cast<unsigned>(t->size); j += nthr) {
      ok = detail::wait_ge_sys(mine + j, epoch, detail::team_pe_to_world(t, j), 60,
                               ROCSHMEM_ERR_BARRIER_TIMEOUT) && ok;
    }
  } else {
    for (unsigned j = tid; j < static_cast<unsigned>(t->size); j += nthr) {
      detail::st_relaxed_sys(detail::remote_ptr(mine + t->my_pe, detail::team_pe_to_world(t, j)), epoch);
    }
    for (unsigned j = tid; j < static_cast<unsigned>(t->size); j += nthr) {
      unsigned long long seen = detail::ld_relaxed_sys(mine + j);
      if (seen < epoch) {
        detail::SpinBudget budget(s.wait_timeout_ns);
        while ((seen = detail::ld_relaxed_sys(mine + j)) < epoch) {
          if (!budget.keep_going()) {
            detail::record_error(ROCSHMEM_ERR_BARRIER_TIMEOUT, detail::team_pe_to_world(t, j), 62, mine + j, epoch, seen);
            ok = false;
            break;
          }
        }
      }
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// Barrier between all blocks of one PE inside a kernel (blocks with the same blockIdx.z). The
// counter only grows; `counter` must be zero before the first use by a kernel instance and every
// block must call it the same number of times (`round` counts the calls, starting at 1). Requires
// all blocks of the PE to be resident (cooperative launch). Returns false on time-out.
__device__ inline bool grid_barrier(unsigned long long *counter, unsigned long long round,
                                    unsigned blocks_per_pe) {
  __syncthreads();
  bool ok = true;
  if (detail::block_tid() == 0) {
    __threadfence();
    atomicAdd(counter, 1ull);
    const unsigned long long target = round * blocks_per_pe;
    detail::SpinBudget budget(st().wait_timeout_ns);
    while (*reinterpret_cast<volatile unsigned long long *>(counter) < target) {
      if (!budget.keep_going()) {
        detail::record_error(ROCSHMEM_ERR_GRID_TIMEOUT, -1, 61, counter, target,
                             *reinterpret_cast<volatile unsigned long long *>(counter));
        ok = false;
        break;
      }
    }
    __threadfence();
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// ---- 16-byte vector helpers ---------------------------------------------------------------------------

template <typename T>
struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

__device__ __forceinline__ int4 ld_global_16(const void *p) { return *reinterpret_cast<const int4 *>(p); }
__device__ __forceinline__ void st_global_16(void *p, int4 v) { *reinterpret_cast<int4 *>(p) = v; }

}  // namespace kernels
}  // namespace rocshmem
