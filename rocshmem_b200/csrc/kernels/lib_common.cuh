// Building blocks shared by the library's own multi-block kernels (collectives, MoE dispatch and
// combine, fused GEMM + collective): block-paired cross-PE barriers, an intra-kernel grid barrier,
// launch helpers that understand several PEs per process.
#pragma once

#include <cuda_runtime.h>

#include "rocshmem/rocshmem.h"

namespace rocshmem {
namespace kernels {

using detail::st;

// Cross-PE barrier between "the same block" on every member of a team: block b of a PE signals
// block b of every member and waits for all of them. Blocks of one PE never wait for each other, so
// a kernel built on this needs no grid-wide synchronisation and no cooperative launch when each PE
// has its own GPU. All members must launch the same number of blocks for the same sequence of
// library calls on a team, which keeps the per-(team, block) epochs in step without communication.
// Returns false if a peer did not arrive within the wait budget (error record written).
__device__ inline bool block_pair_barrier(const rocshmem_team_dev *t, unsigned block) {
  __shared__ unsigned long long s_epoch;
  const rocshmem_device_state &s = st();
  const unsigned tid = detail::block_tid(), nthr = detail::block_threads();
  __syncthreads();
  if (tid == 0) {
    unsigned long long *e = s.lib_state + size_t(t->slot) * ROCSHMEM_LIB_MAX_BLOCKS + block;
    s_epoch = *e + 1;
    *e = s_epoch;
  }
  __syncthreads();
  const unsigned long long epoch = s_epoch;
  unsigned long long *mine =
      s.lib_flags + (size_t(t->slot) * ROCSHMEM_LIB_MAX_BLOCKS + block) * ROCSHMEM_MAX_PES;
  for (unsigned j = tid; j < static_cast<unsigned>(t->size); j += nthr) {
    detail::st_release_sys(detail::remote_ptr(mine + t->my_pe, detail::team_pe_to_world(t, j)), epoch);
  }
  bool ok = true;
  for (unsigned j = tid; j < static_cast<unsigned>(t->size); j += nthr) {
    ok = detail::wait_ge_sys(mine + j, epoch, detail::team_pe_to_world(t, j), 60,
                             ROCSHMEM_ERR_BARRIER_TIMEOUT) && ok;
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
