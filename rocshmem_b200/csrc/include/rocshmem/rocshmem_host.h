// Host-side entry points of the runtime library (librocshmem_b200.so), untyped.
//
// The public, typed names (rocshmem_float_put, rocshmem_int64_atomic_fetch_add, ...) are thin inline
// wrappers over these functions and live in rocshmem.h. Reference counterpart: the host half of
// src/rocshmem.cpp (lines 103-303 and the *_GEN instantiations at 821-1353) forwarding into
// HostInterface (src/host/host.cpp, host_templates.hpp).
#pragma once

#include <stddef.h>
#include <stdint.h>

#include "rocshmem_common.h"

namespace rocshmem {

// Element types understood by the untyped engine (values match rocshmem::DType in the runtime).
enum rocshmem_dtype : int {
  ROCSHMEM_I8 = 0, ROCSHMEM_U8, ROCSHMEM_I16, ROCSHMEM_U16, ROCSHMEM_I32, ROCSHMEM_U32,
  ROCSHMEM_I64, ROCSHMEM_U64, ROCSHMEM_F32, ROCSHMEM_F64, ROCSHMEM_F16, ROCSHMEM_BF16
};

enum rocshmem_amo_op : int {
  ROCSHMEM_AMO_FETCH = 0, ROCSHMEM_AMO_SWAP, ROCSHMEM_AMO_CAS, ROCSHMEM_AMO_ADD,
  ROCSHMEM_AMO_AND, ROCSHMEM_AMO_OR, ROCSHMEM_AMO_XOR
};

extern rocshmem_team_t ROCSHMEM_TEAM_WORLD;

namespace host {

// ---- lifecycle ------------------------------------------------------------------------------
// Bootstraps from the environment: RANK / WORLD_SIZE / LOCAL_RANK as set by torchrun (a single
// process when unset), rendezvous through files under ROCSHMEM_BOOTSTRAP_DIR (by default a directory in
// /dev/shm named after the user, MASTER_PORT, the run id and the launching process, so that every launch
// gets its own; ranks started by different parent processes must set the variable), ROCSHMEM_LOCAL_PES
// PEs per process. Python programs initialise through rocshmem_b200.init() instead, which hands a
// torch.distributed store to the runtime.
void init();
void init_thread(int requested, int *provided);
void query_thread(int *provided);
void finalize();
void global_exit(int status);
bool is_initialized();
int my_pe();   // usable before init (reads RANK), as the reference allows
int n_pes();
void dump_stats();
void reset_stats();

// ---- heap -----------------------------------------------------------------------------------
void *malloc(size_t bytes);
void free(void *ptr);
// Address of the symmetric object `ptr` on `pe` in this process's address space (every peer heap is
// mapped), or nullptr when ptr is not symmetric. The result is a device address on the CUDA
// backend: usable in kernels and cudaMemcpy, not dereferenceable by the CPU.
void *ptr(const void *ptr, int pe);

// ---- contexts and teams ------------------------------------------------------------------------
int ctx_create(int64_t options, rocshmem_ctx_t *ctx);
int team_create_ctx(rocshmem_team_t team, int64_t options, rocshmem_ctx_t *ctx);
void ctx_destroy(rocshmem_ctx_t ctx);
int team_translate_pe(rocshmem_team_t src_team, int src_pe, rocshmem_team_t dst_team);
int team_n_pes(rocshmem_team_t team);
int team_my_pe(rocshmem_team_t team);
int team_split_strided(rocshmem_team_t parent, int start, int stride, int size,
                       const rocshmem_team_config_t *config, long config_mask,
                       rocshmem_team_t *new_team);
void team_destroy(rocshmem_team_t team);

// ---- RMA --------------------------------------------------------------------------------------
void putmem(rocshmem_ctx_t ctx, void *dest, const void *source, size_t bytes, int pe);
void getmem(rocshmem_ctx_t ctx, void *dest, const void *source, size_t bytes, int pe);
void putmem_nbi(rocshmem_ctx_t ctx, void *dest, const void *source, size_t bytes, int pe);
void getmem_nbi(rocshmem_ctx_t ctx, void *dest, const void *source, size_t bytes, int pe);
// Single-element put/get by value (bits of a 1/2/4/8-byte element).
void p(rocshmem_ctx_t ctx, void *dest, uint64_t bits, size_t elem_bytes, int pe);
uint64_t g(rocshmem_ctx_t ctx, const void *source, size_t elem_bytes, int pe);

// ---- atomics ----------------------------------------------------------------------------------
uint64_t amo(rocshmem_ctx_t ctx, int op, int dtype, void *target, uint64_t value, uint64_t cond,
             int pe);

// ---- ordering and synchronisation ------------------------------------------------------------------
void fence(rocshmem_ctx_t ctx);
void quiet(rocshmem_ctx_t ctx);
void barrier_all();
void sync_all();
int team_sync(rocshmem_team_t team);

// wait_until family on a local symmetric variable of type `dtype`. `value` / `values` carry the
// bits of the comparison operand(s). All waits are bounded by ROCSHMEM_WAIT_TIMEOUT_MS; when the
// budget runs out an error record is written and the call returns (SIZE_MAX for any/some).
int wait_until(void *ivar, int dtype, int cmp, uint64_t value);
int test(void *ivar, int dtype, int cmp, uint64_t value);
void wait_until_all(void *ivars, size_t nelems, const int *status, int dtype, int cmp,
                    const uint64_t *values, bool vector);
size_t wait_until_any(void *ivars, size_t nelems, const int *status, int dtype, int cmp,
                      const uint64_t *values, bool vector);
size_t wait_until_some(void *ivars, size_t nelems, size_t *indices, const int *status, int dtype,
                       int cmp, const uint64_t *values, bool vector);

// ---- collectives --------------------------------------------------------------------------------
int broadcast(rocshmem_ctx_t ctx, rocshmem_team_t team, void *dest, const void *source,
              size_t bytes, int pe_root);
int reduce(rocshmem_ctx_t ctx, rocshmem_team_t team, void *dest, const void *source, size_t nreduce,
           int dtype, int op);
int fcollect(rocshmem_ctx_t ctx, rocshmem_team_t team, void *dest, const void *source, size_t bytes);
int alltoall(rocshmem_ctx_t ctx, rocshmem_team_t team, void *dest, const void *source, size_t bytes);
// Active-set forms (PE_start, logPE_stride, PE_size): a temporary team is derived per call.
int broadcast_active_set(rocshmem_ctx_t ctx, void *dest, const void *source, size_t bytes,
                         int pe_root, int pe_start, int log_pe_stride, int pe_size);
int reduce_active_set(rocshmem_ctx_t ctx, void *dest, const void *source, size_t nreduce, int dtype,
                      int op, int pe_start, int log_pe_stride, int pe_size);

}  // namespace host

// ---- extensions (rocshmemx_*) ---------------------------------------------------------------------
// Several PEs per process on one GPU: choose which local PE subsequent host calls of this thread
// act for. Collective calls (malloc, free, team split, barrier_all, collectives) are made once per
// process and act for all its local PEs.
void rocshmemx_set_local_pe(int local_index);
int rocshmemx_n_local_pes();
// First error recorded by a bounded wait / debug check on this PE (kind == 0: none).
rocshmem_error_record rocshmemx_get_error();
void rocshmemx_clear_error();
void rocshmemx_set_wait_timeout_ms(uint64_t ms);
// Copies between ordinary host memory and the symmetric heap (the heap is GPU memory and cannot be
// dereferenced by CPU code; the reference's examples write to it directly).
void rocshmemx_heap_write(void *heap_dst, const void *host_src, size_t bytes);
void rocshmemx_heap_read(void *host_dst, const void *heap_src, size_t bytes);
// Stream used by the default host context (cudaStream_t), for ordering user kernels against
// host-API operations.
void *rocshmemx_default_stream();

}  // namespace rocshmem
