// Host-callable launchers of the library's CUDA kernels. Plain C++ (no CUDA syntax), so the host
// runtime, the Python bindings and C++ user programs can all call them. Pointers to symmetric memory
// are the addresses on the calling process's first local PE; `stream` is a cudaStream_t.
// Every launcher returns 0 on success or a cudaError_t value.
#pragma once

#include <cstddef>
#include <cstdint>

#include "rocshmem/rocshmem_common.h"
#include "rocshmem/rocshmem_host.h"

namespace rocshmem {
namespace kernels {

enum AllreduceAlgo : int {
  ALLREDUCE_AUTO = 0,
  ALLREDUCE_ONE_SHOT = 1,  // every PE reads every source; lowest latency for small payloads
  ALLREDUCE_TWO_SHOT = 2,  // reduce-scatter by pull + all-gather by push; bandwidth-optimal over P2P
  ALLREDUCE_NVLS = 3,      // multimem.ld_reduce + multimem.st through the NVSwitch (TEAM_WORLD only)
  ALLREDUCE_LL = 4,        // up to 2 KiB: data and call number in one 8-byte word, no barrier, one NVLink crossing
};

// ---- collectives on the symmetric heap (coll_kernels.cu) -----------------------------------------------
// Loads every collective kernel of the library now (see coll_kernels.cu); 0 or the first CUDA error.
int coll_preload();
int coll_barrier(rocshmem_team_t team, void *stream);
int coll_allreduce(rocshmem_team_t team, void *dest, const void *source, size_t nelems, int dtype,
                   int op, int algo, void *stream);
// flags: COLL_PRE_SYNC adds a barrier at kernel entry, so that no member writes into a destination
// that another member's earlier stream work may still be reading. Without it the OpenSHMEM rule
// applies: the caller guarantees that every member's dest is ready when the collective starts.
enum CollFlags : int { COLL_NONE = 0, COLL_PRE_SYNC = 1 };
int coll_broadcast(rocshmem_team_t team, void *dest, const void *source, size_t bytes, int root,
                   void *stream, int flags = COLL_NONE);
int coll_fcollect(rocshmem_team_t team, void *dest, const void *source, size_t bytes, void *stream,
                  int flags = COLL_NONE);
int coll_alltoall(rocshmem_team_t team, void *dest, const void *source, size_t bytes, void *stream,
                  int flags = COLL_NONE);
// Number of blocks per PE the collective would use for this payload (exposed for tests).
int coll_blocks_for(size_t bytes);
bool nvls_available();

// ---- helpers for the host API engine (host_kernels.cu) ---------------------------------------------------
// result: device-accessible 8-byte slot that receives the previous value.
int host_amo(int op, int dtype, void *target, uint64_t value, uint64_t cond, uint64_t *result, void *stream);

}  // namespace kernels
}  // namespace rocshmem
