// Kernels of the functional test-suite: user-style __global__ code that calls the device API, in
// the way the reference's functional tester classes do (tests/functional_tests/*_tester.cpp), plus
// the pybind11 glue that launches them. Oracles follow those testers: patterns written
// by the initiator, exact signal counts, max fetched values of atomics, collectives against a host
// reference.
//
// Every kernel receives symmetric addresses as they are on the process's first local PE and rebases
// them with rocshmemx_local(), so the same launch serves one PE per process (gridDim.z == 1) and
// several PEs per process (gridDim.z == n_local, cooperative launch).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cuda_runtime.h>

#include "kernels/launch.cuh"
#include "rocshmem/rocshmem.h"

namespace py = pybind11;
using namespace rocshmem;

namespace {

enum RmaOp { RMA_PUT = 0, RMA_PUT_NBI, RMA_GET, RMA_GET_NBI, RMA_P, RMA_G };
enum ScopeSel { SC_THREAD = 0, SC_WARP, SC_BLOCK };

// Each PE moves `bytes` bytes between its `src` and `dst` on PE (me + shift) % n. With thread scope
// every thread moves its own contiguous share; with warp scope every warp; with block scope the
// block moves everything. Ends with a barrier so the host may verify right after the kernel.
__global__ void rma_kernel(int op, int scope, char *dst_a, const char *src_a, size_t bytes, int shift,
                           int use_ctx) {
  __shared__ rocshmem_ctx_t ctx;
  char *dst = rocshmemx_local(dst_a);
  const char *src = rocshmemx_local(const_cast<char *>(src_a));
  rocshmem_wg_init();
  if (use_ctx) {
    rocshmem_wg_ctx_create(0, &ctx);
  } else {
    if (threadIdx.x == 0) ctx = ROCSHMEM_CTX_DEFAULT;
    __syncthreads();
  }
  const int me = rocshmem_my_pe(), n = rocshmem_n_pes();
  const int pe = (me + shift) % n;
  size_t groups = 1, gid = 0;
  if (scope == SC_THREAD) { groups = blockDim.x; gid = threadIdx.x; }
  if (scope == SC_WARP) { groups = (blockDim.x + 31) / 32; gid = threadIdx.x / 32; }
  size_t share = (bytes + groups - 1) / groups;
  size_t lo = share * gid, hi = lo + share;
  if (lo > bytes) lo = bytes;
  if (hi > bytes) hi = bytes;
  const size_t len = hi - lo;
  switch (op * 3 + scope) {
    case RMA_PUT * 3 + SC_THREAD: rocshmem_ctx_putmem(ctx, dst + lo, src + lo, len, pe); break;
    case RMA_PUT * 3 + SC_WARP: rocshmem_ctx_putmem_warp(ctx, dst + lo, src + lo, len, pe); break;
    case RMA_PUT * 3 + SC_BLOCK: rocshmem_ctx_putmem_block(ctx, dst + lo, src + lo, len, pe); break;
    case RMA_PUT_NBI * 3 + SC_THREAD: rocshmem_ctx_putmem_nbi(ctx, dst + lo, src + lo, len, pe); rocshmem_ctx_quiet(ctx); break;
    case RMA_PUT_NBI * 3 + SC_WARP: rocshmem_ctx_putmem_nbi_wave(ctx, dst + lo, src + lo, len, pe); rocshmem_ctx_quiet(ctx); break;
    case RMA_PUT_NBI * 3 + SC_BLOCK: rocshmem_ctx_putmem_nbi_wg(ctx, dst + lo, src + lo, len, pe); rocshmem_ctx_quiet(ctx); break;
    case RMA_GET * 3 + SC_THREAD: rocshmem_ctx_getmem(ctx, dst + lo, src + lo, len, pe); break;
    case RMA_GET * 3 + SC_WARP: rocshmem_ctx_getmem_wave(ctx, dst + lo, src + lo, len, pe); break;
    case RMA_GET * 3 + SC_BLOCK: rocshmem_ctx_getmem_wg(ctx, dst + lo, src + lo, len, pe); break;
    case RMA_GET_NBI * 3 + SC_THREAD: rocshmem_ctx_getmem_nbi(ctx, dst + lo, src + lo, len, pe); rocshmem_ctx_quiet(ctx); break;
    case RMA_GET_NBI * 3 + SC_WARP: rocshmem_ctx_getmem_nbi_warp(ctx, dst + lo, src + lo, len, pe); rocshmem_ctx_quiet(ctx); break;
    case RMA_GET_NBI * 3 + SC_BLOCK: rocshmem_ctx_getmem_nbi_block(ctx, dst + lo, src + lo, len, pe); rocshmem_ctx_quiet(ctx); break;
    case RMA_P * 3 + SC_THREAD: {
      // element-wise: 8-byte elements
      long long *d = reinterpret_cast<long long *>(dst);
      const long long *s = reinterpret_cast<const long long *>(src);
      for (size_t i = threadIdx.x; i < bytes / 8; i += blockDim.x) rocshmem_ctx_longlong_p(ctx, d + i, s[i], pe);
      break;
    }
    case RMA_G * 3 + SC_THREAD: {
      long long *d = reinterpret_cast<long long *>(dst);
      const long long *s = reinterpret_cast<const long long *>(src);
      for (size_t i = threadIdx.x; i < bytes / 8; i += blockDim.x) d[i] = rocshmem_ctx_longlong_g(ctx, s + i, pe);
      break;
    }
    default: break;
  }
  if (use_ctx) rocshmem_wg_ctx_destroy(&ctx);
  rocshmem_wg_barrier_all();
  rocshmem_wg_finalize();
}

// ---- atomics ------------------------------------------------------------------------------------------
enum AmoTest { A_FADD = 0, A_FINC, A_ADD, A_INC, A_FCSWAP, A_FETCH, A_SET, A_SWAP, A_FAND, A_AND, A_FOR, A_OR, A_FXOR, A_XOR };

// All threads of all PEs hit element 0 of `target` on PE 0, `iters` times each. `ret` (symmetric,
// one slot per thread) records the largest value fetched by that thread.
template <typename T>
__global__ void amo_kernel(int test, T *target_a, T *ret_a, int iters) {
  T *target = rocshmemx_local(target_a);
  T *ret = rocshmemx_local(ret_a);
  T best = 0;
  for (int i = 0; i < iters; ++i) {
    T got = 0;
    switch (test) {
      case A_FADD: got = rocshmem_ctx_int64_atomic_fetch_add(ROCSHMEM_CTX_DEFAULT, (int64_t *)target, 2, 0); break;
      case A_FINC: got = rocshmem_int64_atomic_fetch_inc((int64_t *)target, 0); break;
      case A_ADD: rocshmem_int64_atomic_add((int64_t *)target, 2, 0); break;
      case A_INC: rocshmem_int64_atomic_inc((int64_t *)target, 0); break;
      case A_FCSWAP: {
        // Classic CAS increment: succeeds exactly once per attempt that observed the current value.
        int64_t cur = rocshmem_int64_atomic_fetch((int64_t *)target, 0);
        for (int tries = 0; tries < 100000; ++tries) {
          int64_t seen = rocshmem_int64_atomic_compare_swap((int64_t *)target, cur, cur + 1, 0);
          if (seen == cur) { got = cur; break; }
          cur = seen;
        }
        break;
      }
      case A_FETCH: got = rocshmem_int64_atomic_fetch((int64_t *)target, 0); break;
      case A_SET: rocshmem_int64_atomic_set((int64_t *)target, 44, 0); break;
      case A_SWAP: got = rocshmem_int64_atomic_swap((int64_t *)target, (int64_t)(rocshmem_my_pe() + 1), 0); break;
      case A_FAND: got = rocshmem_int64_atomic_fetch_and((int64_t *)target, 0xFFFF, 0); break;
      case A_AND: rocshmem_int64_atomic_and((int64_t *)target, 0xFFFF, 0); break;
      case A_FOR: got = rocshmem_int64_atomic_fetch_or((int64_t *)target, 0xFFFF, 0); break;
      case A_OR: rocshmem_int64_atomic_or((int64_t *)target, 0xFFFF, 0); break;
      case A_FXOR: got = rocshmem_int64_atomic_fetch_xor((int64_t *)target, 0xFFFF, 0); break;
      case A_XOR: rocshmem_int64_atomic_xor((int64_t *)target, 0xFFFF, 0); break;
      default: break;
    }
    if (got > best) best = got;
  }
  ret[blockIdx.x * blockDim.x + threadIdx.x] = best;
  __syncthreads();
  if (blockIdx.x == 0) rocshmem_wg_barrier_all();
}

// 32-bit and floating-point atomics on PE `pe`: out[0..] receive the values fetched.
__global__ void amo_types_kernel(unsigned int *u32_a, float *f32_a, double *f64_a, int *i32_a,
                                 unsigned long long *out_a, int pe) {
  unsigned int *u32 = rocshmemx_local(u32_a);
  float *f32 = rocshmemx_local(f32_a);
  double *f64 = rocshmemx_local(f64_a);
  int *i32 = rocshmemx_local(i32_a);
  unsigned long long *out = rocshmemx_local(out_a);
  if (threadIdx.x == 0 && rocshmem_my_pe() == 0) {
    out[0] = rocshmem_uint_atomic_fetch_add(u32, 7u, pe);           // 0 -> 7
    out[1] = rocshmem_uint32_atomic_fetch_or(u32, 0xF0u, pe);       // 7 -> 0xF7
    out[2] = rocshmem_uint_atomic_compare_swap(u32, 0xF7u, 5u, pe);  // -> 5
    out[3] = rocshmem_uint_atomic_swap(u32, 9u, pe);                // 5 -> 9
    out[4] = rocshmem_uint_atomic_fetch(u32, pe);                   // 9
    rocshmem_float_atomic_set(f32, 1.5f, pe);
    float old = rocshmem_float_atomic_swap(f32, 2.5f, pe);
    out[5] = __float_as_uint(old);                                   // 1.5
    out[6] = __float_as_uint(rocshmem_float_atomic_fetch(f32, pe));  // 2.5
    rocshmem_double_atomic_set(f64, 3.25, pe);
    out[7] = (unsigned long long)__double_as_longlong(rocshmem_double_atomic_fetch(f64, pe));
    out[8] = (unsigned long long)(long long)rocshmem_int_atomic_fetch_add(i32, -3, pe);  // 0 -> -3
    out[9] = (unsigned long long)(long long)rocshmem_int_atomic_fetch_inc(i32, pe);      // -3 -> -2
    out[10] = (unsigned long long)(long long)rocshmem_int32_atomic_fetch_xor(i32, -1, pe);  // -2 -> 1
    out[11] = (unsigned long long)(long long)rocshmem_int_atomic_fetch(i32, pe);            // 1
  }
  __syncthreads();
  rocshmem_wg_barrier_all();
}

// ---- signals ----------------------------------------------------------------------------------------------
// Every PE sends `bytes` to (me + 1) % n with a signal and waits for its own signal from (me - 1).
// With ADD the expected final value is init + number of signalling groups; SET leaves `value`.
__global__ void signal_kernel(int scope, int sig_op, char *dst_a, const char *src_a, size_t bytes,
                              uint64_t *sig_a, uint64_t value, uint64_t expect, uint64_t *fetched_a) {
  char *dst = rocshmemx_local(dst_a);
  const char *src = rocshmemx_local(const_cast<char *>(src_a));
  uint64_t *sig = rocshmemx_local(sig_a);
  uint64_t *fetched = rocshmemx_local(fetched_a);
  const int me = rocshmem_my_pe(), n = rocshmem_n_pes();
  const int pe = (me + 1) % n;
  if (scope == SC_THREAD) {
    size_t share = bytes / blockDim.x;
    rocshmem_putmem_signal(dst + share * threadIdx.x, src + share * threadIdx.x, share, sig, value, sig_op, pe);
  } else if (scope == SC_WARP) {
    size_t warps = blockDim.x / 32, share = bytes / warps, w = threadIdx.x / 32;
    rocshmem_putmem_signal_wave(dst + share * w, src + share * w, share, sig, value, sig_op, pe);
  } else {
    rocshmem_putmem_signal_wg(dst, src, bytes, sig, value, sig_op, pe);
  }
  if (threadIdx.x == 0) {
    int rc = rocshmemx_uint64_wait_until_status(sig, ROCSHMEM_CMP_EQ, expect);
    fetched[0] = rocshmem_signal_fetch(sig);
    fetched[1] = (uint64_t)rc;
  }
  __syncthreads();
  rocshmem_wg_barrier_all();
}

// ---- ping-pong, ping-all, wait variants -------------------------------------------------------------------------
__global__ void pingpong_kernel(int *flag_a, int iters, long long *cycles_a) {
  int *flag = rocshmemx_local(flag_a);
  long long *cycles = rocshmemx_local(cycles_a);
  const int me = rocshmem_my_pe();
  if (threadIdx.x == 0 && me < 2) {
    unsigned long long t0 = detail::now_ns();
    for (int i = 0; i < iters; ++i) {
      if (me == 0) {
        rocshmem_int_p(flag, i + 1, 1);
        if (rocshmemx_int_wait_until_status(flag, ROCSHMEM_CMP_EQ, i + 1) != ROCSHMEM_SUCCESS) break;
      } else {
        if (rocshmemx_int_wait_until_status(flag, ROCSHMEM_CMP_EQ, i + 1) != ROCSHMEM_SUCCESS) break;
        rocshmem_int_p(flag, i + 1, 0);
      }
    }
    cycles[0] = (long long)(detail::now_ns() - t0);
  }
  __syncthreads();
  rocshmem_wg_barrier_all();
}

// Every PE writes 1 into slot[me] on all PEs, then waits for all of its slots with wait_until_all;
// then exercises any / some / vector forms and test. result[] receives the observations.
__global__ void pingall_kernel(long *slots_a, long long *result_a) {
  long *slots = rocshmemx_local(slots_a);
  long long *result = rocshmemx_local(result_a);
  const int me = rocshmem_my_pe(), n = rocshmem_n_pes();
  if (threadIdx.x == 0) {
    for (int j = 0; j < n; ++j) rocshmem_long_p(slots + me, (long)(me + 1), j);
    long vals[ROCSHMEM_MAX_PES];
    int status[ROCSHMEM_MAX_PES];
    size_t idx[ROCSHMEM_MAX_PES];
    for (int j = 0; j < n; ++j) { vals[j] = j + 1; status[j] = 0; }
    rocshmem_long_wait_until_all(slots, n, nullptr, ROCSHMEM_CMP_GE, 1);
    rocshmem_long_wait_until_all_vector(slots, n, status, ROCSHMEM_CMP_EQ, vals);
    result[0] = (long long)rocshmem_long_wait_until_any(slots, n, nullptr, ROCSHMEM_CMP_EQ, (long)n);   // index n-1
    result[1] = (long long)rocshmem_long_wait_until_some(slots, n, idx, nullptr, ROCSHMEM_CMP_GT, 0);   // n
    status[0] = 1;  // mask slot 0
    result[2] = (long long)rocshmem_long_wait_until_any_vector(slots, n, status, ROCSHMEM_CMP_EQ, vals); // 1 (or SIZE_MAX if n==1)
    result[3] = (long long)rocshmem_long_wait_until_some_vector(slots, n, idx, status, ROCSHMEM_CMP_EQ, vals);  // n-1
    result[4] = rocshmem_long_test(slots + me, ROCSHMEM_CMP_NE, 0);   // 1
    result[5] = rocshmem_long_test(slots + me, ROCSHMEM_CMP_LT, 0);   // 0
    result[6] = (long long)rocshmem_long_wait_until_any(slots, 0, nullptr, ROCSHMEM_CMP_EQ, 1);  // SIZE_MAX
    for (int j = 0; j < n; ++j) status[j] = 1;
    result[7] = (long long)rocshmem_long_wait_until_any(slots, n, status, ROCSHMEM_CMP_EQ, 1);   // SIZE_MAX
  }
  __syncthreads();
  rocshmem_wg_barrier_all();
}

// Waits on a flag nobody sets: the wait must give up and report, leaving the context usable.
__global__ void timeout_kernel(uint64_t *flag_a, int *status_a) {
  uint64_t *flag = rocshmemx_local(flag_a);
  int *status = rocshmemx_local(status_a);
  if (threadIdx.x == 0) status[0] = rocshmemx_uint64_wait_until_status(flag, ROCSHMEM_CMP_EQ, 12345ull);
}

// ---- contexts and teams ------------------------------------------------------------------------------------------------
// out[0] = rc of wg_ctx_create, out[1] = ctx_my_pe, out[2] = ctx_n_pes, out[3] = translate(team, my, world)
// Members put their team rank into slot[team_rank] on every team member through a team context
// (team-relative PE numbers), then team-sync.
__global__ void team_ctx_kernel(rocshmem_team_t team, rocshmem_team_t world, int *slots_a, int *out_a) {
  __shared__ rocshmem_ctx_t ctx;
  int *slots = rocshmemx_local(slots_a);
  int *out = rocshmemx_local(out_a);
  const int my = rocshmemx_team_my_pe(team);
  if (my < 0) {
    if (threadIdx.x == 0) out[0] = -2;
    return;
  }
  int rc = rocshmem_wg_team_create_ctx(team, 0, &ctx);
  if (threadIdx.x == 0) {
    out[0] = rc;
    out[1] = rocshmem_ctx_my_pe(ctx);
    out[2] = rocshmem_ctx_n_pes(ctx);
    out[3] = rocshmem_team_translate_pe(team, my, world);
    const int n = rocshmem_ctx_n_pes(ctx);
    for (int j = 0; j < n; ++j) rocshmem_ctx_int_p(ctx, slots + my, my + 100, j);
  }
  rocshmem_wg_ctx_destroy(&ctx);
  rocshmem_wg_team_sync(team);
}

// Takes `want` contexts in one block and reports how many creations succeeded.
__global__ void ctx_exhaust_kernel(int want, int *out_a) {
  __shared__ rocshmem_ctx_t ctx[64];
  int *out = rocshmemx_local(out_a);
  int ok = 0;
  for (int i = 0; i < want && i < 64; ++i) {
    if (rocshmem_wg_ctx_create(0, &ctx[i]) == 0) ++ok;
  }
  if (threadIdx.x == 0) out[0] = ok;
  for (int i = 0; i < want && i < 64; ++i) rocshmem_wg_ctx_destroy(&ctx[i]);
}

// ---- block collectives --------------------------------------------------------------------------------------------------------
enum CollOp { C_BCAST = 0, C_FCOLLECT, C_ALLTOALL, C_SUM, C_MIN, C_MAX, C_PROD, C_AND, C_OR, C_XOR };

template <typename T>
__device__ int run_reduce(int op, rocshmem_team_t team, T *dst, const T *src, int n);

#define RUN_REDUCE_ARITH(T, N)                                                                    \
  template <>                                                                                     \
  __device__ int run_reduce<T>(int op, rocshmem_team_t team, T *dst, const T *src, int n) {       \
    switch (op) {                                                                                 \
      case C_SUM: return rocshmem_ctx_##N##_sum_wg_reduce(ROCSHMEM_CTX_DEFAULT, team, dst, src, n);  \
      case C_MIN: return rocshmem_ctx_##N##_min_wg_reduce(ROCSHMEM_CTX_DEFAULT, team, dst, src, n);  \
      case C_MAX: return rocshmem_ctx_##N##_max_wg_reduce(ROCSHMEM_CTX_DEFAULT, team, dst, src, n);  \
      case C_PROD: return rocshmem_ctx_##N##_prod_block_reduce(ROCSHMEM_CTX_DEFAULT, team, dst, src, n); \
      default: return run_reduce_bitwise<T>(op, team, dst, src, n);                               \
    }                                                                                             \
  }
template <typename T>
__device__ int run_reduce_bitwise(int, rocshmem_team_t, T *, const T *, int) { return -1; }
#define RUN_REDUCE_BITWISE(T, N)                                                                  \
  template <>                                                                                     \
  __device__ int run_reduce_bitwise<T>(int op, rocshmem_team_t team, T *dst, const T *src, int n) { \
    switch (op) {                                                                                 \
      case C_AND: return rocshmem_ctx_##N##_and_wg_reduce(ROCSHMEM_CTX_DEFAULT, team, dst, src, n);  \
      case C_OR: return rocshmem_ctx_##N##_or_wg_reduce(ROCSHMEM_CTX_DEFAULT, team, dst, src, n);    \
      case C_XOR: return rocshmem_ctx_##N##_xor_block_reduce(ROCSHMEM_CTX_DEFAULT, team, dst, src, n); \
      default: return -1;                                                                         \
    }                                                                                             \
  }
RUN_REDUCE_BITWISE(short, short)
RUN_REDUCE_BITWISE(int, int)
RUN_REDUCE_BITWISE(long, long)
RUN_REDUCE_BITWISE(long long, longlong)
RUN_REDUCE_ARITH(short, short)
RUN_REDUCE_ARITH(int, int)
RUN_REDUCE_ARITH(long, long)
RUN_REDUCE_ARITH(long long, longlong)
RUN_REDUCE_ARITH(float, float)
RUN_REDUCE_ARITH(double, double)
RUN_REDUCE_ARITH(__half, half)
RUN_REDUCE_ARITH(__nv_bfloat16, bfloat16)

template <typename T>
__device__ void run_copy_coll(int op, rocshmem_team_t team, T *dst, const T *src, int n, int root);
#define RUN_COPY_COLL(T, N)                                                                       \
  template <>                                                                                     \
  __device__ void run_copy_coll<T>(int op, rocshmem_team_t team, T *dst, const T *src, int n, int root) { \
    if (op == C_BCAST) rocshmem_ctx_##N##_wg_broadcast(ROCSHMEM_CTX_DEFAULT, team, dst, src, n, root);   \
    if (op == C_FCOLLECT) rocshmem_ctx_##N##_wg_fcollect(ROCSHMEM_CTX_DEFAULT, team, dst, src, n);       \
    if (op == C_ALLTOALL) rocshmem_ctx_##N##_block_alltoall(ROCSHMEM_CTX_DEFAULT, team, dst, src, n);    \
  }
RUN_COPY_COLL(float, float)
RUN_COPY_COLL(double, double)
RUN_COPY_COLL(char, char)
RUN_COPY_COLL(short, short)
RUN_COPY_COLL(int, int)
RUN_COPY_COLL(long, long)
RUN_COPY_COLL(long long, longlong)
template <> __device__ void run_copy_coll<__half>(int, rocshmem_team_t, __half *, const __half *, int, int) {}
template <> __device__ void run_copy_coll<__nv_bfloat16>(int, rocshmem_team_t, __nv_bfloat16 *, const __nv_bfloat16 *, int, int) {}
template <> __device__ int run_reduce<char>(int, rocshmem_team_t, char *, const char *, int) { return -1; }

// One block per PE runs one block-collective on `team` `repeat` times (back-to-back use of the same
// team exercises the epoch logic), then a barrier.
template <typename T>
__global__ void coll_kernel(int op, rocshmem_team_t team, T *dst_a, const T *src_a, int nelems, int root,
                            int repeat, int *rc_a) {
  T *dst = rocshmemx_local(dst_a);
  const T *src = rocshmemx_local(const_cast<T *>(src_a));
  int *rc = rocshmemx_local(rc_a);
  if (rocshmemx_team_my_pe(team) < 0) return;
  int r = 0;
  for (int i = 0; i < repeat; ++i) {
    if (op >= C_SUM) r |= run_reduce<T>(op, team, dst, src, nelems);
    else run_copy_coll<T>(op, team, dst, src, nelems, root);
  }
  if (threadIdx.x == 0) rc[0] = r;
  rocshmem_wg_team_sync(team);
}

// ---- barrier stress, shmem_ptr, local copy alignment --------------------------------------------------------------------------
// Round r: every PE writes r into slot[me] on every PE, barrier, then checks that all slots hold r.
__global__ void barrier_kernel(long long *slots_a, int rounds, int *errors_a) {
  long long *slots = rocshmemx_local(slots_a);
  int *errors = rocshmemx_local(errors_a);
  const int me = rocshmem_my_pe(), n = rocshmem_n_pes();
  int bad = 0;
  for (int r = 1; r <= rounds; ++r) {
    for (int j = threadIdx.x; j < n; j += blockDim.x) rocshmem_longlong_p(slots + me, (long long)r, j);
    if (r & 1) rocshmem_wg_barrier_all(); else rocshmem_wg_sync_all();
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
      if (*reinterpret_cast<volatile long long *>(slots + j) < r) ++bad;
    }
    rocshmem_wg_barrier_all();
  }
  atomicAdd(errors, bad);
}

__global__ void ptr_kernel(char *buf_a, int offset) {
  char *buf = rocshmemx_local(buf_a);
  const int me = rocshmem_my_pe(), n = rocshmem_n_pes();
  if (threadIdx.x == 0) {
    char *peer = static_cast<char *>(rocshmem_ptr(buf, (me + 1) % n));
    if (peer != nullptr) peer[offset] = (char)('1' + me);
    if (rocshmem_ptr(buf, n) != nullptr) buf[0] = 'X';  // out-of-range PE must give nullptr
  }
  __syncthreads();
  rocshmem_wg_barrier_all();
}

// Local copies (pe == me) of every size/alignment combination requested, with all three scopes.
__global__ void copy_align_kernel(int scope, char *dst_a, const char *src_a, int max_len, int max_align) {
  char *dst = rocshmemx_local(dst_a);
  const char *src = rocshmemx_local(const_cast<char *>(src_a));
  const int me = rocshmem_my_pe();
  // case index -> (len, src offset, dst offset); each case has its own 256-byte aligned slot pair
  const int stride = ((max_len + 2 * max_align + 255) / 256) * 256;
  int c = 0;
  for (int len = 0; len <= max_len; ++len) {
    for (int so = 0; so < max_align; so += (so < 4 ? 1 : 5)) {
      for (int d_o = 0; d_o < max_align; d_o += (d_o < 4 ? 1 : 7)) {
        char *d = dst + size_t(c) * stride + d_o;
        const char *s = src + size_t(c) * stride + so;
        if (scope == SC_THREAD) { if (threadIdx.x == 0) rocshmem_putmem(d, s, len, me); }
        else if (scope == SC_WARP) { if (threadIdx.x < 32) rocshmem_putmem_wave(d, s, len, me); }
        else rocshmem_putmem_wg(d, s, len, me);
        ++c;
      }
    }
  }
}

// ---- bandwidth / latency probes (device-timed) ------------------------------------------------------------------------------------
// PE 0 moves `bytes` to/from PE `pe` `iters` times with `blocks` blocks; elapsed nanoseconds per
// block are written to ns[]. mode: 0 put_nbi_block + quiet, 1 get_block, 2 put_signal_block + peer wait.
__global__ void bw_kernel(int mode, char *dst_a, const char *src_a, size_t bytes, int pe, int iters,
                          unsigned long long *ns_a) {
  char *dst = rocshmemx_local(dst_a);
  const char *src = rocshmemx_local(const_cast<char *>(src_a));
  unsigned long long *ns = rocshmemx_local(ns_a);
  if (rocshmem_my_pe() != 0) return;
  size_t share = ((bytes + gridDim.x - 1) / gridDim.x + 15) / 16 * 16;
  size_t lo = share * blockIdx.x, hi = lo + share;
  if (lo > bytes) lo = bytes;
  if (hi > bytes) hi = bytes;
  __syncthreads();
  unsigned long long t0 = detail::now_ns();
  for (int i = 0; i < iters; ++i) {
    if (mode == 0) {
      rocshmem_putmem_nbi_wg(dst + lo, src + lo, hi - lo, pe);
    } else {
      rocshmem_getmem_wg(dst + lo, src + lo, hi - lo, pe);
    }
  }
  rocshmem_quiet();
  __syncthreads();
  if (threadIdx.x == 0) ns[blockIdx.x] = detail::now_ns() - t0;
}

// Micro-benchmark of the device API (the reference's primitive / message-rate / atomic testers:
// tests/functional_tests/primitive_tester.cpp, primitive_mr_tester.cpp:41-52, amo_standard_tester.cpp:82-100).
// Every active PE runs `iters` rounds; in round i it talks to PE (me + 1 + i % (n - 1)) % n when `all_pairs` is set
// (every PE targets every other in turn) and to its successor otherwise; with all_pairs == 0 only PE 0 is active
// (a pair of PEs), except for the put-with-signal ring, which needs every PE.
//   op 0 put (blocking)   1 get   2 window of 64 put_nbi + quiet (message rate)   3 put_signal to the successor,
//   then wait_until on my own signal (one hop of a ring per round)   4 int64 fetch_add   5 int64 compare_swap
// `groups` thread / warp / block groups of the grid take part, each moving its own slice of `bytes` (atomics: one
// operation per participating thread). Elapsed nanoseconds of every block go to ns[blockIdx.x].
enum BenchOp { B_PUT = 0, B_GET, B_PUT_NBI_WINDOW, B_PUT_SIGNAL_RING, B_FETCH_ADD, B_COMPARE_SWAP };

__global__ void rma_bench_kernel(int op, int scope, char *dst_a, const char *src_a, size_t bytes, int groups,
                                 int iters, int all_pairs, uint64_t *sig_a, long long *counter_a,
                                 unsigned long long *ns_a, uint64_t sig_base) {
  char *dst = rocshmemx_local(dst_a);
  const char *src = rocshmemx_local(const_cast<char *>(src_a));
  uint64_t *sig = rocshmemx_local(sig_a);
  long long *counter = rocshmemx_local(counter_a);
  unsigned long long *ns = rocshmemx_local(ns_a);
  const int me = rocshmem_my_pe(), n = rocshmem_n_pes();
  const bool ring = op == B_PUT_SIGNAL_RING;
  if (n < 2 || (!all_pairs && !ring && me != 0)) return;
  // Which group am I, and does it take part?
  int gid, per_block;
  if (scope == SC_THREAD) { per_block = blockDim.x; gid = blockIdx.x * per_block + threadIdx.x; }
  else if (scope == SC_WARP) { per_block = blockDim.x / 32; gid = blockIdx.x * per_block + threadIdx.x / 32; }
  else { per_block = 1; gid = blockIdx.x; }
  const bool active = gid < groups;
  size_t share = ((bytes + groups - 1) / groups + 15) / 16 * 16;
  if (bytes < 16) share = bytes;
  size_t lo = share * size_t(gid), hi = lo + share;
  if (lo > bytes) lo = bytes;
  if (hi > bytes) hi = bytes;
  const size_t len = active ? hi - lo : 0;
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const unsigned long long t0 = detail::now_ns();
  for (int i = 0; i < iters; ++i) {
    const int pe = all_pairs ? (me + 1 + i % (n - 1)) % n : (me + 1) % n;
    if (op == B_PUT || op == B_GET) {
      if (active) {
        if (scope == SC_THREAD) {
          if (op == B_PUT) rocshmem_putmem(dst + lo, src + lo, len, pe); else rocshmem_getmem(dst + lo, src + lo, len, pe);
        } else if (scope == SC_WARP) {
          if (op == B_PUT) rocshmem_putmem_wave(dst + lo, src + lo, len, pe); else rocshmem_getmem_wave(dst + lo, src + lo, len, pe);
        } else {
          if (op == B_PUT) rocshmem_putmem_wg(dst + lo, src + lo, len, pe); else rocshmem_getmem_wg(dst + lo, src + lo, len, pe);
        }
      }
    } else if (op == B_PUT_NBI_WINDOW) {
      if (active) {
        for (int m = 0; m < 64; ++m) {
          if (scope == SC_THREAD) rocshmem_putmem_nbi(dst + lo, src + lo, len, pe);
          else if (scope == SC_WARP) rocshmem_putmem_nbi_wave(dst + lo, src + lo, len, pe);
          else rocshmem_putmem_nbi_wg(dst + lo, src + lo, len, pe);
        }
        rocshmem_quiet();
      }
    } else if (ring) {
      // One group only (the host passes groups == 1): group 0 of block 0.
      if (blockIdx.x == 0 && gid == 0) {
        const uint64_t value = sig_base + uint64_t(i) + 1;
        const int next = (me + 1) % n;
        if (scope == SC_THREAD) {
          if (threadIdx.x == 0) rocshmem_putmem_signal(dst, src, bytes, sig, value, ROCSHMEM_SIGNAL_SET, next);
        } else if (scope == SC_WARP) {
          rocshmem_putmem_signal_wave(dst, src, bytes, sig, value, ROCSHMEM_SIGNAL_SET, next);
        } else {
          rocshmem_putmem_signal_wg(dst, src, bytes, sig, value, ROCSHMEM_SIGNAL_SET, next);
        }
        // A wait that ran out ends the loop for the whole group at once (the calls above are collective).
        if (threadIdx.x == 0 && rocshmemx_uint64_wait_until_status(sig, ROCSHMEM_CMP_GE, value) != ROCSHMEM_SUCCESS) {
          s_fail = 1;
        }
        if (scope == SC_BLOCK) __syncthreads();
        else if (scope == SC_WARP) __syncwarp();
        if (*reinterpret_cast<volatile int *>(&s_fail)) break;
      }
    } else if (active) {
      if (op == B_FETCH_ADD) {
        (void)rocshmem_longlong_atomic_fetch_add(counter, 1, pe);
      } else {
        (void)rocshmem_longlong_atomic_compare_swap(counter, (long long)i, (long long)i + 1, pe);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) ns[blockIdx.x] = detail::now_ns() - t0;
}

// Compile-time coverage of the typed API surface: references one member of every generated family
// for every type table entry. It is launched with run == 0, so nothing executes.
__global__ void api_surface_kernel(int run, void *p, rocshmem_team_t team) {
  if (!run) return;
  rocshmem_ctx_t c = ROCSHMEM_CTX_DEFAULT;
#define SURF_RMA(T, N)                                                                           \
  rocshmem_ctx_##N##_put(c, (T *)p, (const T *)p, 0, 0); rocshmem_##N##_get((T *)p, (const T *)p, 0, 0); \
  rocshmem_##N##_put_nbi((T *)p, (const T *)p, 0, 0); rocshmem_ctx_##N##_get_nbi(c, (T *)p, (const T *)p, 0, 0); \
  rocshmem_##N##_p((T *)p, (T)0, 0); (void)rocshmem_ctx_##N##_g(c, (const T *)p, 0);              \
  rocshmem_##N##_put_wave((T *)p, (const T *)p, 0, 0); rocshmem_ctx_##N##_put_wg(c, (T *)p, (const T *)p, 0, 0); \
  rocshmem_##N##_get_warp((T *)p, (const T *)p, 0, 0); rocshmem_##N##_get_block((T *)p, (const T *)p, 0, 0); \
  rocshmem_##N##_put_nbi_wave((T *)p, (const T *)p, 0, 0); rocshmem_##N##_get_nbi_wg((T *)p, (const T *)p, 0, 0);
  ROCSHMEM_RMA_TYPES(SURF_RMA)
#define SURF_SIG(T, N)                                                                           \
  rocshmem_##N##_put_signal((T *)p, (const T *)p, 0, (uint64_t *)p, 0, 0, 0);                     \
  rocshmem_ctx_##N##_put_signal_wg(c, (T *)p, (const T *)p, 0, (uint64_t *)p, 0, 0, 0);           \
  rocshmem_##N##_put_signal_nbi_wave((T *)p, (const T *)p, 0, (uint64_t *)p, 0, 0, 0);            \
  rocshmem_ctx_##N##_wg_broadcast(c, team, (T *)p, (const T *)p, 0, 0);                           \
  rocshmem_ctx_##N##_wg_alltoall(c, team, (T *)p, (const T *)p, 0);                               \
  rocshmem_ctx_##N##_wg_fcollect(c, team, (T *)p, (const T *)p, 0);
  ROCSHMEM_STANDARD_RMA_TYPES(SURF_SIG)
#define SURF_AMO(T, N, D)                                                                        \
  (void)rocshmem_##N##_atomic_fetch((T *)p, 0); rocshmem_ctx_##N##_atomic_set(c, (T *)p, (T)0, 0); \
  (void)rocshmem_##N##_atomic_swap((T *)p, (T)0, 0);
  ROCSHMEM_AMO_STANDARD_TYPES(SURF_AMO)
  ROCSHMEM_AMO_EXTENDED_ONLY_TYPES(SURF_AMO)
#define SURF_AMO_STD(T, N, D)                                                                    \
  (void)rocshmem_##N##_atomic_compare_swap((T *)p, (T)0, (T)0, 0); (void)rocshmem_##N##_atomic_fetch_inc((T *)p, 0); \
  rocshmem_##N##_atomic_inc((T *)p, 0); (void)rocshmem_ctx_##N##_atomic_fetch_add(c, (T *)p, (T)0, 0); \
  rocshmem_##N##_atomic_add((T *)p, (T)0, 0);
  ROCSHMEM_AMO_STANDARD_TYPES(SURF_AMO_STD)
#define SURF_AMO_BIT(T, N, D)                                                                    \
  (void)rocshmem_##N##_atomic_fetch_and((T *)p, (T)0, 0); rocshmem_##N##_atomic_and((T *)p, (T)0, 0); \
  (void)rocshmem_##N##_atomic_fetch_or((T *)p, (T)0, 0); rocshmem_##N##_atomic_or((T *)p, (T)0, 0);   \
  (void)rocshmem_##N##_atomic_fetch_xor((T *)p, (T)0, 0); rocshmem_ctx_##N##_atomic_xor(c, (T *)p, (T)0, 0);
  ROCSHMEM_AMO_BITWISE_TYPES(SURF_AMO_BIT)
#define SURF_SYNC(T, N, D)                                                                       \
  rocshmem_##N##_wait_until((T *)p, 0, (T)0); (void)rocshmem_##N##_test((T *)p, 0, (T)0);          \
  rocshmem_##N##_wait_until_all((T *)p, 0, nullptr, 0, (T)0);                                     \
  (void)rocshmem_##N##_wait_until_any((T *)p, 0, nullptr, 0, (T)0);                               \
  (void)rocshmem_##N##_wait_until_some((T *)p, 0, nullptr, nullptr, 0, (T)0);                     \
  rocshmem_##N##_wait_until_all_vector((T *)p, 0, nullptr, 0, (T *)p);                            \
  (void)rocshmem_##N##_wait_until_any_vector((T *)p, 0, nullptr, 0, (T *)p);                      \
  (void)rocshmem_##N##_wait_until_some_vector((T *)p, 0, nullptr, nullptr, 0, (T *)p);
  ROCSHMEM_SYNC_TYPES(SURF_SYNC)
  rocshmem_fence(); rocshmem_fence(0); rocshmem_ctx_fence(c, 0); rocshmem_quiet(); rocshmem_threadfence_system();
  rocshmem_ctx_threadfence_system(c); (void)rocshmem_signal_fetch_wg((uint64_t *)p);
  (void)rocshmem_signal_fetch_wave((uint64_t *)p); int prov; rocshmem_query_thread(&prov); rocshmem_wg_init_thread(0, &prov);
}

// Every block adds to a plain (non-atomic) counter `rounds` times under the ticket lock and as many times
// under the spin lock (thread 0 only); a grid barrier separates two phases whose order the host checks.
__global__ void mutex_kernel(rocshmemx_ticket_mutex_t *ticket, rocshmemx_spin_mutex_t *spin, unsigned long long *counters,
                             unsigned long long *grid_counter, int rounds, int *phase_errors) {
  for (int r = 0; r < rounds; ++r) {
    if (!rocshmemx_ticket_lock_block(ticket)) return;
    if (threadIdx.x == 0) {
      volatile unsigned long long *c = counters;
      *c = *c + 1;
    }
    rocshmemx_ticket_unlock_block(ticket);
  }
  if (threadIdx.x == 0) {
    for (int r = 0; r < rounds; ++r) {
      if (!rocshmemx_spin_lock(spin)) return;
      volatile unsigned long long *c = counters + 1;
      *c = *c + 1;
      rocshmemx_spin_unlock(spin);
    }
  }
  if (!rocshmemx_grid_sync(grid_counter, 1, gridDim.x)) return;
  // After the barrier every block must see all increments of the first phase.
  if (threadIdx.x == 0) {
    const unsigned long long want = static_cast<unsigned long long>(gridDim.x) * rounds;
    if (*reinterpret_cast<volatile unsigned long long *>(counters) != want) atomicAdd(phase_errors, 1);
    if (*reinterpret_cast<volatile unsigned long long *>(counters + 1) != want) atomicAdd(phase_errors, 1);
  }
}

// Slab allocation from device code. Every thread allocates `bytes` (16-byte aligned) and records its pointer; then
// every warp allocates once for its lanes and every block once for its threads, and each thread checks that it saw
// the same pointer as lane 0 / thread 0 (differences are counted in `errors`).
__global__ void slab_kernel(rocshmemx_slab_t slab, size_t bytes, unsigned long long *thread_ptrs,
                            unsigned long long *warp_ptrs, unsigned long long *block_ptrs, int *errors) {
  const unsigned g = blockIdx.x * blockDim.x + threadIdx.x;
  void *p = rocshmemx_slab_alloc(slab, bytes, 16);
  thread_ptrs[g] = reinterpret_cast<unsigned long long>(p);
  if (p != nullptr) *static_cast<unsigned int *>(p) = g;   // the block is usable memory
  __syncwarp();  // the lanes left the compare-and-swap loop above at different times: converge before a warp-level call
  void *w = rocshmemx_slab_alloc_wave(slab, 64, 64);
  const unsigned long long w0 = __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(w), 0);
  if (w0 != reinterpret_cast<unsigned long long>(w)) atomicAdd(errors, 1);
  if ((threadIdx.x & 31) == 0) warp_ptrs[g / 32] = reinterpret_cast<unsigned long long>(w);
  void *b = rocshmemx_slab_alloc_wg(slab, 256, 256);
  __shared__ unsigned long long first;
  if (threadIdx.x == 0) first = reinterpret_cast<unsigned long long>(b);
  __syncthreads();
  if (first != reinterpret_cast<unsigned long long>(b)) atomicAdd(errors, 1);
  if (threadIdx.x == 0) block_ptrs[blockIdx.x] = first;
}

// ---- launch glue ---------------------------------------------------------------------------------------------------------------------

template <typename T> T *P(uintptr_t v) { return reinterpret_cast<T *>(v); }
cudaStream_t S(uintptr_t s) { return reinterpret_cast<cudaStream_t>(s); }
void ok(cudaError_t e, const char *what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

template <typename T>
void launch_coll_t(int op, uintptr_t team, uintptr_t dst, uintptr_t src, int n, int root, int repeat,
                   uintptr_t rc, int threads, uintptr_t stream) {
  ok(kernels::launch_pes(coll_kernel<T>, 1, threads, 0, S(stream), false, op,
                         reinterpret_cast<rocshmem_team_t>(team), P<T>(dst), P<T>(src), n, root, repeat,
                         P<int>(rc)), "coll_kernel");
}

}  // namespace

PYBIND11_MODULE(_testk, m) {
  m.def("rma", [](int op, int scope, uintptr_t dst, uintptr_t src, size_t bytes, int shift, int use_ctx,
                  int threads, uintptr_t stream) {
    ok(kernels::launch_pes(rma_kernel, 1, threads, 0, S(stream), false, op, scope, P<char>(dst),
                           P<char>(src), bytes, shift, use_ctx), "rma_kernel");
  });
  m.def("amo", [](int test, uintptr_t target, uintptr_t ret, int iters, int blocks, int threads, uintptr_t stream) {
    ok(kernels::launch_pes(amo_kernel<long long>, blocks, threads, 0, S(stream), false, test,
                           P<long long>(target), P<long long>(ret), iters), "amo_kernel");
  });
  m.def("amo_types", [](uintptr_t u32, uintptr_t f32, uintptr_t f64, uintptr_t i32, uintptr_t out, int pe,
                        uintptr_t stream) {
    ok(kernels::launch_pes(amo_types_kernel, 1, 32, 0, S(stream), false, P<unsigned int>(u32), P<float>(f32),
                           P<double>(f64), P<int>(i32), P<unsigned long long>(out), pe), "amo_types_kernel");
  });
  m.def("signal", [](int scope, int sig_op, uintptr_t dst, uintptr_t src, size_t bytes, uintptr_t sig,
                     uint64_t value, uint64_t expect, uintptr_t fetched, int threads, uintptr_t stream) {
    ok(kernels::launch_pes(signal_kernel, 1, threads, 0, S(stream), false, scope, sig_op, P<char>(dst),
                           P<char>(src), bytes, P<uint64_t>(sig), value, expect, P<uint64_t>(fetched)),
       "signal_kernel");
  });
  m.def("pingpong", [](uintptr_t flag, int iters, uintptr_t ns, uintptr_t stream) {
    ok(kernels::launch_pes(pingpong_kernel, 1, 32, 0, S(stream), false, P<int>(flag), iters, P<long long>(ns)),
       "pingpong_kernel");
  });
  m.def("pingall", [](uintptr_t slots, uintptr_t result, uintptr_t stream) {
    ok(kernels::launch_pes(pingall_kernel, 1, 32, 0, S(stream), false, P<long>(slots), P<long long>(result)),
       "pingall_kernel");
  });
  m.def("timeout", [](uintptr_t flag, uintptr_t status, uintptr_t stream) {
    ok(kernels::launch_pes(timeout_kernel, 1, 32, 0, S(stream), false, P<uint64_t>(flag), P<int>(status)),
       "timeout_kernel");
  });
  m.def("team_ctx", [](uintptr_t team, uintptr_t world, uintptr_t slots, uintptr_t out, uintptr_t stream) {
    ok(kernels::launch_pes(team_ctx_kernel, 1, 64, 0, S(stream), false,
                           reinterpret_cast<rocshmem_team_t>(team), reinterpret_cast<rocshmem_team_t>(world),
                           P<int>(slots), P<int>(out)), "team_ctx_kernel");
  });
  m.def("ctx_exhaust", [](int want, uintptr_t out, uintptr_t stream) {
    ok(kernels::launch_pes(ctx_exhaust_kernel, 1, 32, 0, S(stream), false, want, P<int>(out)), "ctx_exhaust_kernel");
  });
  m.def("coll", [](int op, const std::string &dtype, uintptr_t team, uintptr_t dst, uintptr_t src, int n, int root,
                   int repeat, uintptr_t rc, int threads, uintptr_t stream) {
    if (dtype == "float32") launch_coll_t<float>(op, team, dst, src, n, root, repeat, rc, threads, stream);
    else if (dtype == "float64") launch_coll_t<double>(op, team, dst, src, n, root, repeat, rc, threads, stream);
    else if (dtype == "int16") launch_coll_t<short>(op, team, dst, src, n, root, repeat, rc, threads, stream);
    else if (dtype == "int32") launch_coll_t<int>(op, team, dst, src, n, root, repeat, rc, threads, stream);
    else if (dtype == "int64") launch_coll_t<long long>(op, team, dst, src, n, root, repeat, rc, threads, stream);
    else if (dtype == "long") launch_coll_t<long>(op, team, dst, src, n, root, repeat, rc, threads, stream);
    else if (dtype == "int8") launch_coll_t<char>(op, team, dst, src, n, root, repeat, rc, threads, stream);
    else if (dtype == "float16") launch_coll_t<__half>(op, team, dst, src, n, root, repeat, rc, threads, stream);
    else if (dtype == "bfloat16") launch_coll_t<__nv_bfloat16>(op, team, dst, src, n, root, repeat, rc, threads, stream);
    else throw std::invalid_argument("coll: dtype");
  });
  m.def("barrier_stress", [](uintptr_t slots, int rounds, uintptr_t errors, int threads, uintptr_t stream) {
    ok(kernels::launch_pes(barrier_kernel, 1, threads, 0, S(stream), false, P<long long>(slots), rounds,
                           P<int>(errors)), "barrier_kernel");
  });
  m.def("shmem_ptr", [](uintptr_t buf, int offset, uintptr_t stream) {
    ok(kernels::launch_pes(ptr_kernel, 1, 32, 0, S(stream), false, P<char>(buf), offset), "ptr_kernel");
  });
  m.def("copy_align", [](int scope, uintptr_t dst, uintptr_t src, int max_len, int max_align, int threads,
                         uintptr_t stream) {
    ok(kernels::launch_pes(copy_align_kernel, 1, threads, 0, S(stream), false, scope, P<char>(dst), P<char>(src),
                           max_len, max_align), "copy_align_kernel");
  });
  m.def("bw", [](int mode, uintptr_t dst, uintptr_t src, size_t bytes, int pe, int iters, uintptr_t ns, int blocks,
                 int threads, uintptr_t stream) {
    ok(kernels::launch_pes(bw_kernel, blocks, threads, 0, S(stream), false, mode, P<char>(dst), P<char>(src),
                           bytes, pe, iters, P<unsigned long long>(ns)), "bw_kernel");
  });
  m.def("rma_bench", [](int op, int scope, uintptr_t dst, uintptr_t src, size_t bytes, int groups, int iters,
                        int all_pairs, uintptr_t sig, uintptr_t counter, uintptr_t ns, uint64_t sig_base, int blocks,
                        int threads, uintptr_t stream) {
    ok(kernels::launch_pes(rma_bench_kernel, blocks, threads, 0, S(stream), false, op, scope, P<char>(dst),
                           P<char>(src), bytes, groups, iters, all_pairs, P<uint64_t>(sig), P<long long>(counter),
                           P<unsigned long long>(ns), sig_base), "rma_bench_kernel");
  });
  m.def("mutex_test", [](uintptr_t ticket, uintptr_t spin, uintptr_t counters, uintptr_t grid_counter, int rounds,
                         uintptr_t phase_errors, int blocks, int threads, uintptr_t stream) {
    mutex_kernel<<<blocks, threads, 0, S(stream)>>>(P<rocshmemx_ticket_mutex_t>(ticket), P<rocshmemx_spin_mutex_t>(spin),
                                                    P<unsigned long long>(counters), P<unsigned long long>(grid_counter),
                                                    rounds, P<int>(phase_errors));
    ok(cudaGetLastError(), "mutex_kernel");
  });
  m.def("slab_test", [](uintptr_t base, uint64_t size, size_t bytes, uintptr_t thread_ptrs, uintptr_t warp_ptrs,
                        uintptr_t block_ptrs, uintptr_t errors, int blocks, int threads, uintptr_t stream) {
    rocshmemx_slab_t slab{reinterpret_cast<char *>(base), size, reinterpret_cast<unsigned long long *>(base + size)};
    slab_kernel<<<blocks, threads, 0, S(stream)>>>(slab, bytes, P<unsigned long long>(thread_ptrs),
                                                   P<unsigned long long>(warp_ptrs), P<unsigned long long>(block_ptrs),
                                                   P<int>(errors));
    ok(cudaGetLastError(), "slab_kernel");
  });
  m.def("api_surface", [](uintptr_t p, uintptr_t team, uintptr_t stream) {
    ok(kernels::launch_pes(api_surface_kernel, 1, 32, 0, S(stream), false, 0, P<void>(p),
                           reinterpret_cast<rocshmem_team_t>(team)), "api_surface_kernel");
  });
}
