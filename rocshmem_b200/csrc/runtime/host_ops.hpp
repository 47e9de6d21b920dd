// Engine behind the host-side API: how a put/get/atomic/wait/collective issued from CPU code is
// carried out against the mapped window.
//
// The reference implements the whole host API on MPI-3 one-sided windows over the heap
// (src/host/host.hpp:102-401, host_templates.hpp): MPI_Put/MPI_Get + MPI_Win_flush for RMA,
// MPI_Fetch_and_op / MPI_Compare_and_swap for atomics, MPI_Bcast / MPI_Allreduce for collectives,
// polling MPI_Fetch_and_op(NO_OP) for wait_until. There is no MPI here:
//   * CudaHostOps (host_ops_cuda.cu): stream-ordered copies on the peer-mapped addresses and small
//     helper kernels that perform the atomic / wait / barrier / collective on the GPU, so host- and
//     device-initiated operations meet in the same memory with the same (.sys scope) semantics. A
//     host context owns one stream: that stream is its ordering and completion domain, quiet is a
//     stream synchronise.
//   * CpuHostOps (host_ops_cpu.cpp): the same contract on the shared-memory heap, with C++ atomics.
#pragma once

#include <cstddef>
#include <cstdint>

#include "rocshmem/rocshmem_common.h"

namespace rocshmem {

struct HostCtx;
struct HostTeam;
class Runtime;

enum class DType : int { I8 = 0, U8, I16, U16, I32, U32, I64, U64, F32, F64, F16, BF16 };
size_t dtype_size(DType t);
bool dtype_is_float(DType t);
bool dtype_is_signed(DType t);

// Every atomic returns the previous value; the non-fetching API variants discard it.
enum class AmoOp : int { FETCH = 0, SWAP, CAS, ADD, AND, OR, XOR };

class HostOps {
 public:
  virtual ~HostOps() = default;

  // dst/src are addresses valid on the initiating PE; `remote_*` marks which one is symmetric and
  // has to be translated to `pe` (put: dst, get: src).
  virtual void put(HostCtx *ctx, void *dst, const void *src, size_t bytes, int pe, bool blocking) = 0;
  virtual void get(HostCtx *ctx, void *dst, const void *src, size_t bytes, int pe, bool blocking) = 0;
  virtual uint64_t amo(HostCtx *ctx, AmoOp op, DType t, void *target, uint64_t value, uint64_t cond,
                       int pe) = 0;
  virtual void fence(HostCtx *ctx) = 0;
  virtual void quiet(HostCtx *ctx) = 0;
  // 1 when `*ivar cmp value` holds now, else 0.
  virtual int test(void *ivar, DType t, int cmp, uint64_t value) = 0;
  // ROCSHMEM_SUCCESS, or ROCSHMEM_ERROR after the configured time-out (an error record is written).
  virtual int wait_until(void *ivar, DType t, int cmp, uint64_t value) = 0;

  // Team collectives; the caller has validated membership. `sync_only` skips the quiet.
  virtual int barrier(HostCtx *ctx, HostTeam *team, bool sync_only) = 0;
  virtual int broadcast(HostCtx *ctx, HostTeam *team, void *dst, const void *src, size_t bytes,
                        int root) = 0;
  virtual int reduce(HostCtx *ctx, HostTeam *team, void *dst, const void *src, size_t nelems,
                     DType t, ROCSHMEM_OP op) = 0;
  virtual int fcollect(HostCtx *ctx, HostTeam *team, void *dst, const void *src, size_t bytes) = 0;
  virtual int alltoall(HostCtx *ctx, HostTeam *team, void *dst, const void *src, size_t bytes) = 0;

  // Context resources (a stream on CUDA).
  virtual void ctx_init(HostCtx *ctx) = 0;
  virtual void ctx_fini(HostCtx *ctx) = 0;
};

HostOps *make_cpu_host_ops(Runtime *rt);
HostOps *make_cuda_host_ops(Runtime *rt);

// Compare helper shared by the CPU engine and tests: interprets the raw bits as type t.
bool compare_bits(uint64_t observed, DType t, int cmp, uint64_t value);

}  // namespace rocshmem
