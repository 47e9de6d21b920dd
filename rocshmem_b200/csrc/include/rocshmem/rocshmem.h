// Public API: OpenSHMEM-style free functions in namespace rocshmem, host and device.
//
// Same names, argument order and semantics as the reference's public headers
// (include/rocshmem/rocshmem.hpp, rocshmem_RMA.hpp, rocshmem_RMA_X.hpp, rocshmem_AMO.hpp,
// rocshmem_SIG_OP.hpp, rocshmem_P2P_SYNC.hpp, rocshmem_COLL.hpp). The reference expands ~6 kLoC of
// prototypes with a Python generator (utils/header_files_gen); here the same surface is produced
// by X-macro type tables in this one header, and rocshmem_b200/utils/gen_api.py lists the expanded
// names from the same tables for documentation and tests.
//
// Compiled by a plain C++ compiler this header gives the host API. Compiled by nvcc every function
// that exists on both sides is __host__ __device__ and picks its implementation by compilation
// pass; device-only families (warp / block RMA, signals, block collectives) are __device__.
// Granularity suffixes are _warp and _block; the reference's _wave and _wg spellings are kept as
// aliases so existing kernels compile unchanged (a "wave" is the 32-lane warp here).
//
// Deliberate differences from the reference, all documented where they occur:
//   * context-based calls translate the team-relative PE for every family (the reference skips the
//     translation for wave/wg RMA, atomics and signals, src/rocshmem_gpu.cpp:641-913);
//   * rocshmem_ptr returns a usable peer address (the reference's IPC backend returns nullptr);
//   * all atomic families are implemented; *_vector waits take an array of values and work;
//   * waits are bounded (ROCSHMEM_WAIT_TIMEOUT_MS) and report through rocshmemx_get_error();
//   * CPU code cannot dereference rocshmem_malloc memory (it is GPU memory): use
//     rocshmemx_heap_write / rocshmemx_heap_read, cudaMemcpy, or the PyTorch symmetric tensors.
#pragma once

#include "rocshmem_common.h"
#include "rocshmem_host.h"
#include "slab.h"

#if defined(__CUDACC__)
#include "device/collectives.cuh"
#include "device/sync.cuh"
#define ROCSHMEM_API __host__ __device__ inline
#define ROCSHMEM_DEVICE_API __device__ inline
#else
#define ROCSHMEM_API inline
#endif

namespace rocshmem {

// The default context. A zero handle selects it on both host and device (TEAM_WORLD numbering).
// The names expand to a function call so that they work unqualified, qualified with rocshmem::,
// in host code and in device code alike.
ROCSHMEM_API rocshmem_ctx_t rocshmem_default_ctx() { return rocshmem_ctx_t{nullptr, nullptr}; }
#define ROCSHMEM_CTX_DEFAULT rocshmem_default_ctx()
#define ROCSHMEM_HOST_CTX_DEFAULT rocshmem_default_ctx()

// ---------------------------------------------------------------------------------------------------
// Type tables: X(c_type, api_name)
// ---------------------------------------------------------------------------------------------------
#define ROCSHMEM_STANDARD_RMA_TYPES(X)                                                           \
  X(float, float) X(double, double) X(char, char) X(signed char, schar) X(short, short)           \
  X(int, int) X(long, long) X(long long, longlong) X(unsigned char, uchar)                        \
  X(unsigned short, ushort) X(unsigned int, uint) X(unsigned long, ulong)                         \
  X(unsigned long long, ulonglong)
#define ROCSHMEM_FIXED_RMA_TYPES(X)                                                              \
  X(int8_t, int8) X(int16_t, int16) X(int32_t, int32) X(int64_t, int64) X(uint8_t, uint8)         \
  X(uint16_t, uint16) X(uint32_t, uint32) X(uint64_t, uint64) X(size_t, size) X(ptrdiff_t, ptrdiff)
#define ROCSHMEM_RMA_TYPES(X) ROCSHMEM_STANDARD_RMA_TYPES(X) ROCSHMEM_FIXED_RMA_TYPES(X)

#define ROCSHMEM_AMO_STANDARD_TYPES(X)                                                           \
  X(int, int, ROCSHMEM_I32) X(long, long, ROCSHMEM_I64) X(long long, longlong, ROCSHMEM_I64)      \
  X(unsigned int, uint, ROCSHMEM_U32) X(unsigned long, ulong, ROCSHMEM_U64)                       \
  X(unsigned long long, ulonglong, ROCSHMEM_U64) X(int32_t, int32, ROCSHMEM_I32)                  \
  X(int64_t, int64, ROCSHMEM_I64) X(uint32_t, uint32, ROCSHMEM_U32) X(uint64_t, uint64, ROCSHMEM_U64) \
  X(size_t, size, ROCSHMEM_U64) X(ptrdiff_t, ptrdiff, ROCSHMEM_I64)
#define ROCSHMEM_AMO_EXTENDED_ONLY_TYPES(X) X(float, float, ROCSHMEM_F32) X(double, double, ROCSHMEM_F64)
#define ROCSHMEM_AMO_BITWISE_TYPES(X)                                                            \
  X(unsigned int, uint, ROCSHMEM_U32) X(unsigned long, ulong, ROCSHMEM_U64)                       \
  X(unsigned long long, ulonglong, ROCSHMEM_U64) X(int32_t, int32, ROCSHMEM_I32)                  \
  X(int64_t, int64, ROCSHMEM_I64) X(uint32_t, uint32, ROCSHMEM_U32) X(uint64_t, uint64, ROCSHMEM_U64)

// Wait/test types with the engine's element code.
#define ROCSHMEM_SYNC_TYPES(X)                                                                   \
  X(float, float, ROCSHMEM_F32) X(double, double, ROCSHMEM_F64) X(char, char, ROCSHMEM_I8)        \
  X(signed char, schar, ROCSHMEM_I8) X(short, short, ROCSHMEM_I16) X(int, int, ROCSHMEM_I32)      \
  X(long, long, ROCSHMEM_I64) X(long long, longlong, ROCSHMEM_I64) X(unsigned char, uchar, ROCSHMEM_U8) \
  X(unsigned short, ushort, ROCSHMEM_U16) X(unsigned int, uint, ROCSHMEM_U32)                     \
  X(unsigned long, ulong, ROCSHMEM_U64) X(unsigned long long, ulonglong, ROCSHMEM_U64)            \
  X(int32_t, int32, ROCSHMEM_I32) X(int64_t, int64, ROCSHMEM_I64) X(uint32_t, uint32, ROCSHMEM_U32) \
  X(uint64_t, uint64, ROCSHMEM_U64) X(size_t, size, ROCSHMEM_U64) X(ptrdiff_t, ptrdiff, ROCSHMEM_I64)

// Reduction tables: X(c_type, api_name, dtype_code)
#define ROCSHMEM_REDUCE_INT_TYPES(X)                                                             \
  X(short, short, ROCSHMEM_I16) X(int, int, ROCSHMEM_I32) X(long, long, ROCSHMEM_I64)             \
  X(long long, longlong, ROCSHMEM_I64)
#define ROCSHMEM_REDUCE_FLOAT_TYPES(X) X(float, float, ROCSHMEM_F32) X(double, double, ROCSHMEM_F64)

namespace api_detail {
template <typename T>
inline uint64_t bits_of(T v) {
  uint64_t b = 0;
  __builtin_memcpy(&b, &v, sizeof(T));
  return b;
}
template <typename T>
inline T value_of(uint64_t b) {
  T v;
  __builtin_memcpy(&v, &b, sizeof(T));
  return v;
}
}  // namespace api_detail

// ===================================================================================================
// Lifecycle, identity, heap, contexts, teams, ordering
// ===================================================================================================

inline void rocshmem_init() { host::init(); }
inline void rocshmem_init_thread(int requested, int *provided) { host::init_thread(requested, provided); }
inline void rocshmem_finalize() { host::finalize(); }
inline void rocshmem_global_exit(int status) { host::global_exit(status); }
inline void rocshmem_dump_stats() { host::dump_stats(); }
inline void rocshmem_reset_stats() { host::reset_stats(); }
inline void *rocshmem_malloc(size_t size) { return host::malloc(size); }
inline void rocshmem_free(void *ptr) { host::free(ptr); }
inline int rocshmem_ctx_create(int64_t options, rocshmem_ctx_t *ctx) { return host::ctx_create(options, ctx); }
inline int rocshmem_team_create_ctx(rocshmem_team_t team, long options, rocshmem_ctx_t *ctx) {
  return host::team_create_ctx(team, options, ctx);
}
inline void rocshmem_ctx_destroy(rocshmem_ctx_t ctx) { host::ctx_destroy(ctx); }
inline int rocshmem_team_n_pes(rocshmem_team_t team) { return host::team_n_pes(team); }
inline int rocshmem_team_my_pe(rocshmem_team_t team) { return host::team_my_pe(team); }
inline int rocshmem_team_split_strided(rocshmem_team_t parent_team, int start, int stride, int size,
                                       const rocshmem_team_config_t *config, long config_mask,
                                       rocshmem_team_t *new_team) {
  return host::team_split_strided(parent_team, start, stride, size, config, config_mask, new_team);
}
inline void rocshmem_team_destroy(rocshmem_team_t team) { host::team_destroy(team); }
inline void rocshmem_barrier_all() { host::barrier_all(); }
inline void rocshmem_sync_all() { host::sync_all(); }
inline int rocshmem_team_sync(rocshmem_team_t team) { return host::team_sync(team); }

ROCSHMEM_API void rocshmem_query_thread(int *provided) {
#if defined(__CUDA_ARCH__)
  *provided = ROCSHMEM_THREAD_MULTIPLE;
#else
  host::query_thread(provided);
#endif
}

ROCSHMEM_API int rocshmem_my_pe() {
#if defined(__CUDA_ARCH__)
  return detail::st().my_pe;
#else
  return host::my_pe();
#endif
}
ROCSHMEM_API int rocshmem_n_pes() {
#if defined(__CUDA_ARCH__)
  return detail::st().n_pes;
#else
  return host::n_pes();
#endif
}
ROCSHMEM_API int rocshmem_team_translate_pe(rocshmem_team_t src_team, int src_pe, rocshmem_team_t dst_team) {
#if defined(__CUDA_ARCH__)
  return detail::team_translate(src_team, src_pe, dst_team);
#else
  return host::team_translate_pe(src_team, src_pe, dst_team);
#endif
}
ROCSHMEM_API void rocshmem_ctx_fence(rocshmem_ctx_t ctx) {
#if defined(__CUDA_ARCH__)
  if (!(detail::ctx_options(ctx) & ROCSHMEM_CTX_NOSTORE)) detail::fence();
  detail::stat_add(ROCSHMEM_STAT_FENCE);
#else
  host::fence(ctx);
#endif
}
ROCSHMEM_API void rocshmem_fence() { rocshmem_ctx_fence(ROCSHMEM_CTX_DEFAULT); }
ROCSHMEM_API void rocshmem_ctx_quiet(rocshmem_ctx_t ctx) {
#if defined(__CUDA_ARCH__)
  (void)ctx;
  detail::quiet();
  detail::stat_add(ROCSHMEM_STAT_QUIET);
#else
  host::quiet(ctx);
#endif
}
ROCSHMEM_API void rocshmem_quiet() { rocshmem_ctx_quiet(ROCSHMEM_CTX_DEFAULT); }
// Peer-addressable pointer to `dest` on `pe`. On the host the result is a device address.
ROCSHMEM_API void *rocshmem_ptr(const void *dest, int pe) {
#if defined(__CUDA_ARCH__)
  if (pe < 0 || pe >= detail::st().n_pes) return nullptr;
  return detail::remote_ptr(static_cast<char *>(const_cast<void *>(dest)), pe);
#else
  return host::ptr(dest, pe);
#endif
}

#if defined(__CUDACC__)
// ---- device-only lifecycle / identity / ordering / sync -------------------------------------------------
ROCSHMEM_DEVICE_API void rocshmem_wg_init() {}
ROCSHMEM_DEVICE_API void rocshmem_wg_finalize() {}
ROCSHMEM_DEVICE_API void rocshmem_wg_init_thread(int, int *provided) { *provided = ROCSHMEM_THREAD_MULTIPLE; }
ROCSHMEM_DEVICE_API int rocshmem_wg_ctx_create(int64_t options, rocshmem_ctx_t *ctx) {
  return detail::ctx_create(options, detail::world_team(), ctx);
}
ROCSHMEM_DEVICE_API int rocshmem_wg_team_create_ctx(rocshmem_team_t team, long options, rocshmem_ctx_t *ctx) {
  if (team == nullptr) return -1;
  return detail::ctx_create(options, detail::team_of(team), ctx);
}
ROCSHMEM_DEVICE_API void rocshmem_wg_ctx_destroy(rocshmem_ctx_t *ctx) { detail::ctx_destroy(ctx); }
ROCSHMEM_DEVICE_API void rocshmem_ctx_fence(rocshmem_ctx_t ctx, int) { rocshmem_ctx_fence(ctx); }
ROCSHMEM_DEVICE_API void rocshmem_fence(int) { rocshmem_fence(); }
ROCSHMEM_DEVICE_API void rocshmem_ctx_threadfence_system(rocshmem_ctx_t) { __threadfence_system(); }
ROCSHMEM_DEVICE_API void rocshmem_threadfence_system() { __threadfence_system(); }
ROCSHMEM_DEVICE_API int rocshmem_ctx_n_pes(rocshmem_ctx_t ctx) { return detail::ctx_team(ctx)->size; }
ROCSHMEM_DEVICE_API int rocshmem_ctx_my_pe(rocshmem_ctx_t ctx) { return detail::ctx_team(ctx)->my_pe; }
// Device-side team queries (extension; the reference offers only translate on the device).
ROCSHMEM_DEVICE_API int rocshmemx_team_my_pe(rocshmem_team_t team) {
  return team == nullptr ? -1 : detail::team_of(team)->my_pe;
}
ROCSHMEM_DEVICE_API int rocshmemx_team_n_pes(rocshmem_team_t team) {
  return team == nullptr ? -1 : detail::team_of(team)->size;
}
// Rebase a symmetric kernel argument to the calling block's PE (identity with one PE per process).
template <typename T>
ROCSHMEM_DEVICE_API T *rocshmemx_local(T *p) { return detail::local_ptr(p); }

// Block-collective: all threads of ONE block per grid (world) or per team call these.
ROCSHMEM_DEVICE_API void rocshmem_ctx_block_barrier_all(rocshmem_ctx_t) {
  detail::stat_add(ROCSHMEM_STAT_BARRIER);
  detail::team_barrier(detail::world_team());
}
ROCSHMEM_DEVICE_API void rocshmem_block_barrier_all() { rocshmem_ctx_block_barrier_all(ROCSHMEM_CTX_DEFAULT); }
ROCSHMEM_DEVICE_API void rocshmem_ctx_block_sync_all(rocshmem_ctx_t) {
  detail::stat_add(ROCSHMEM_STAT_SYNC);
  detail::team_barrier(detail::world_team());
}
ROCSHMEM_DEVICE_API void rocshmem_block_sync_all() { rocshmem_ctx_block_sync_all(ROCSHMEM_CTX_DEFAULT); }
ROCSHMEM_DEVICE_API void rocshmem_ctx_block_team_sync(rocshmem_ctx_t, rocshmem_team_t team) {
  if (team == nullptr) return;
  detail::stat_add(ROCSHMEM_STAT_SYNC);
  detail::team_barrier(detail::team_of(team));
}
ROCSHMEM_DEVICE_API void rocshmem_block_team_sync(rocshmem_team_t team) {
  rocshmem_ctx_block_team_sync(ROCSHMEM_CTX_DEFAULT, team);
}
// Status-returning form (extension): ROCSHMEM_ERROR when a member did not arrive in time.
ROCSHMEM_DEVICE_API int rocshmemx_block_team_sync_status(rocshmem_team_t team) {
  return team == nullptr ? ROCSHMEM_ERROR : detail::team_barrier(detail::team_of(team));
}
ROCSHMEM_DEVICE_API void rocshmem_ctx_wg_barrier_all(rocshmem_ctx_t c) { rocshmem_ctx_block_barrier_all(c); }
ROCSHMEM_DEVICE_API void rocshmem_wg_barrier_all() { rocshmem_block_barrier_all(); }
ROCSHMEM_DEVICE_API void rocshmem_ctx_wg_sync_all(rocshmem_ctx_t c) { rocshmem_ctx_block_sync_all(c); }
ROCSHMEM_DEVICE_API void rocshmem_wg_sync_all() { rocshmem_block_sync_all(); }
ROCSHMEM_DEVICE_API void rocshmem_ctx_wg_team_sync(rocshmem_ctx_t c, rocshmem_team_t t) { rocshmem_ctx_block_team_sync(c, t); }
ROCSHMEM_DEVICE_API void rocshmem_wg_team_sync(rocshmem_team_t t) { rocshmem_block_team_sync(t); }
#endif  // __CUDACC__

// ===================================================================================================
// RMA: thread-level (host + device)
// ===================================================================================================

#if defined(__CUDACC__)
#define ROCSHMEM_DEV_NOSTORE(ctx) ((detail::ctx_options(ctx) & ROCSHMEM_CTX_NOSTORE) != 0)
#endif

ROCSHMEM_API void rocshmem_ctx_putmem(rocshmem_ctx_t ctx, void *dest, const void *source, size_t nelems, int pe) {
#if defined(__CUDA_ARCH__)
  detail::stat_add(ROCSHMEM_STAT_PUT);
  detail::putmem<detail::Scope::THREAD>(dest, source, nelems, detail::ctx_pe(ctx, pe), true, !ROCSHMEM_DEV_NOSTORE(ctx));
#else
  host::putmem(ctx, dest, source, nelems, pe);
#endif
}
ROCSHMEM_API void rocshmem_ctx_getmem(rocshmem_ctx_t ctx, void *dest, const void *source, size_t nelems, int pe) {
#if defined(__CUDA_ARCH__)
  detail::stat_add(ROCSHMEM_STAT_GET);
  detail::getmem<detail::Scope::THREAD>(dest, source, nelems, detail::ctx_pe(ctx, pe), true);
#else
  host::getmem(ctx, dest, source, nelems, pe);
#endif
}
ROCSHMEM_API void rocshmem_ctx_putmem_nbi(rocshmem_ctx_t ctx, void *dest, const void *source, size_t nelems, int pe) {
#if defined(__CUDA_ARCH__)
  detail::stat_add(ROCSHMEM_STAT_PUT_NBI);
  detail::putmem<detail::Scope::THREAD>(dest, source, nelems, detail::ctx_pe(ctx, pe), false, false);
#else
  host::putmem_nbi(ctx, dest, source, nelems, pe);
#endif
}
ROCSHMEM_API void rocshmem_ctx_getmem_nbi(rocshmem_ctx_t ctx, void *dest, const void *source, size_t nelems, int pe) {
#if defined(__CUDA_ARCH__)
  detail::stat_add(ROCSHMEM_STAT_GET_NBI);
  detail::getmem<detail::Scope::THREAD>(dest, source, nelems, detail::ctx_pe(ctx, pe), false);
#else
  host::getmem_nbi(ctx, dest, source, nelems, pe);
#endif
}
ROCSHMEM_API void rocshmem_putmem(void *dest, const void *source, size_t nelems, int pe) {
  rocshmem_ctx_putmem(ROCSHMEM_CTX_DEFAULT, dest, source, nelems, pe);
}
ROCSHMEM_API void rocshmem_getmem(void *dest, const void *source, size_t nelems, int pe) {
  rocshmem_ctx_getmem(ROCSHMEM_CTX_DEFAULT, dest, source, nelems, pe);
}
ROCSHMEM_API void rocshmem_putmem_nbi(void *dest, const void *source, size_t nelems, int pe) {
  rocshmem_ctx_putmem_nbi(ROCSHMEM_CTX_DEFAULT, dest, source, nelems, pe);
}
ROCSHMEM_API void rocshmem_getmem_nbi(void *dest, const void *source, size_t nelems, int pe) {
  rocshmem_ctx_getmem_nbi(ROCSHMEM_CTX_DEFAULT, dest, source, nelems, pe);
}

#if defined(__CUDA_ARCH__)
#define ROCSHMEM_P_BODY(T) detail::stat_add(ROCSHMEM_STAT_P); detail::put_value<T>(dest, value, detail::ctx_pe(ctx, pe));
#define ROCSHMEM_G_BODY(T) detail::stat_add(ROCSHMEM_STAT_G); return detail::get_value<T>(source, detail::ctx_pe(ctx, pe));
#else
#define ROCSHMEM_P_BODY(T) host::p(ctx, dest, api_detail::bits_of<T>(value), sizeof(T), pe);
#define ROCSHMEM_G_BODY(T) return api_detail::value_of<T>(host::g(ctx, source, sizeof(T), pe));
#endif

#define ROCSHMEM_RMA_TYPED(T, N)                                                                   \
  ROCSHMEM_API void rocshmem_ctx_##N##_put(rocshmem_ctx_t ctx, T *dest, const T *source, size_t nelems, int pe) { \
    rocshmem_ctx_putmem(ctx, dest, source, nelems * sizeof(T), pe);                                \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_##N##_put(T *dest, const T *source, size_t nelems, int pe) {          \
    rocshmem_ctx_putmem(ROCSHMEM_CTX_DEFAULT, dest, source, nelems * sizeof(T), pe);               \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_ctx_##N##_get(rocshmem_ctx_t ctx, T *dest, const T *source, size_t nelems, int pe) { \
    rocshmem_ctx_getmem(ctx, dest, source, nelems * sizeof(T), pe);                                \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_##N##_get(T *dest, const T *source, size_t nelems, int pe) {          \
    rocshmem_ctx_getmem(ROCSHMEM_CTX_DEFAULT, dest, source, nelems * sizeof(T), pe);               \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_ctx_##N##_put_nbi(rocshmem_ctx_t ctx, T *dest, const T *source, size_t nelems, int pe) { \
    rocshmem_ctx_putmem_nbi(ctx, dest, source, nelems * sizeof(T), pe);                            \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_##N##_put_nbi(T *dest, const T *source, size_t nelems, int pe) {      \
    rocshmem_ctx_putmem_nbi(ROCSHMEM_CTX_DEFAULT, dest, source, nelems * sizeof(T), pe);           \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_ctx_##N##_get_nbi(rocshmem_ctx_t ctx, T *dest, const T *source, size_t nelems, int pe) { \
    rocshmem_ctx_getmem_nbi(ctx, dest, source, nelems * sizeof(T), pe);                            \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_##N##_get_nbi(T *dest, const T *source, size_t nelems, int pe) {      \
    rocshmem_ctx_getmem_nbi(ROCSHMEM_CTX_DEFAULT, dest, source, nelems * sizeof(T), pe);           \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_ctx_##N##_p(rocshmem_ctx_t ctx, T *dest, T value, int pe) { ROCSHMEM_P_BODY(T) } \
  ROCSHMEM_API void rocshmem_##N##_p(T *dest, T value, int pe) {                                   \
    rocshmem_ctx_##N##_p(ROCSHMEM_CTX_DEFAULT, dest, value, pe);                                   \
  }                                                                                                \
  ROCSHMEM_API T rocshmem_ctx_##N##_g(rocshmem_ctx_t ctx, const T *source, int pe) { ROCSHMEM_G_BODY(T) } \
  ROCSHMEM_API T rocshmem_##N##_g(const T *source, int pe) {                                       \
    return rocshmem_ctx_##N##_g(ROCSHMEM_CTX_DEFAULT, source, pe);                                 \
  }
ROCSHMEM_RMA_TYPES(ROCSHMEM_RMA_TYPED)

// ===================================================================================================
// Atomics (host + device)
// ===================================================================================================

#if defined(__CUDA_ARCH__)
#define ROCSHMEM_AMO_DISPATCH(dev_expr, host_expr) detail::stat_add(ROCSHMEM_STAT_AMO_FETCH); return dev_expr;
#define ROCSHMEM_AMO_DISPATCH_VOID(dev_expr, host_expr) detail::stat_add(ROCSHMEM_STAT_AMO_NOFETCH); dev_expr;
#else
#define ROCSHMEM_AMO_DISPATCH(dev_expr, host_expr) return host_expr;
#define ROCSHMEM_AMO_DISPATCH_VOID(dev_expr, host_expr) (void)host_expr;
#endif
#define ROCSHMEM_HOST_AMO(T, D, OP, target, value, cond)                                           \
  api_detail::value_of<T>(host::amo(ctx, OP, D, const_cast<T *>(target), api_detail::bits_of<T>(value), \
                                    api_detail::bits_of<T>(cond), pe))

// fetch / set / swap: every AMO type including float and double.
#define ROCSHMEM_AMO_EXTENDED(T, N, D)                                                             \
  ROCSHMEM_API T rocshmem_ctx_##N##_atomic_fetch(rocshmem_ctx_t ctx, T *source, int pe) {          \
    ROCSHMEM_AMO_DISPATCH(detail::amo_fetch<T>(source, detail::ctx_pe(ctx, pe)),                   \
                          ROCSHMEM_HOST_AMO(T, D, ROCSHMEM_AMO_FETCH, source, static_cast<T>(0), static_cast<T>(0)))           \
  }                                                                                                \
  ROCSHMEM_API T rocshmem_##N##_atomic_fetch(T *source, int pe) {                                  \
    return rocshmem_ctx_##N##_atomic_fetch(ROCSHMEM_CTX_DEFAULT, source, pe);                      \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_ctx_##N##_atomic_set(rocshmem_ctx_t ctx, T *dest, T value, int pe) {  \
    ROCSHMEM_AMO_DISPATCH_VOID(detail::amo_swap<T>(dest, value, detail::ctx_pe(ctx, pe)),          \
                               ROCSHMEM_HOST_AMO(T, D, ROCSHMEM_AMO_SWAP, dest, value, static_cast<T>(0)))       \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_##N##_atomic_set(T *dest, T value, int pe) {                          \
    rocshmem_ctx_##N##_atomic_set(ROCSHMEM_CTX_DEFAULT, dest, value, pe);                          \
  }                                                                                                \
  ROCSHMEM_API T rocshmem_ctx_##N##_atomic_swap(rocshmem_ctx_t ctx, T *dest, T value, int pe) {    \
    ROCSHMEM_AMO_DISPATCH(detail::amo_swap<T>(dest, value, detail::ctx_pe(ctx, pe)),               \
                          ROCSHMEM_HOST_AMO(T, D, ROCSHMEM_AMO_SWAP, dest, value, static_cast<T>(0)))            \
  }                                                                                                \
  ROCSHMEM_API T rocshmem_##N##_atomic_swap(T *dest, T value, int pe) {                            \
    return rocshmem_ctx_##N##_atomic_swap(ROCSHMEM_CTX_DEFAULT, dest, value, pe);                  \
  }
ROCSHMEM_AMO_STANDARD_TYPES(ROCSHMEM_AMO_EXTENDED)
ROCSHMEM_AMO_EXTENDED_ONLY_TYPES(ROCSHMEM_AMO_EXTENDED)

// compare_swap / fetch_inc / inc / fetch_add / add: integer AMO types.
#define ROCSHMEM_AMO_STANDARD(T, N, D)                                                             \
  ROCSHMEM_API T rocshmem_ctx_##N##_atomic_compare_swap(rocshmem_ctx_t ctx, T *dest, T cond, T value, int pe) { \
    ROCSHMEM_AMO_DISPATCH(detail::amo_cas<T>(dest, cond, value, detail::ctx_pe(ctx, pe)),          \
                          ROCSHMEM_HOST_AMO(T, D, ROCSHMEM_AMO_CAS, dest, value, cond))            \
  }                                                                                                \
  ROCSHMEM_API T rocshmem_##N##_atomic_compare_swap(T *dest, T cond, T value, int pe) {            \
    return rocshmem_ctx_##N##_atomic_compare_swap(ROCSHMEM_CTX_DEFAULT, dest, cond, value, pe);    \
  }                                                                                                \
  ROCSHMEM_API T rocshmem_ctx_##N##_atomic_fetch_add(rocshmem_ctx_t ctx, T *dest, T value, int pe) { \
    ROCSHMEM_AMO_DISPATCH(detail::amo_fetch_add<T>(dest, value, detail::ctx_pe(ctx, pe)),          \
                          ROCSHMEM_HOST_AMO(T, D, ROCSHMEM_AMO_ADD, dest, value, static_cast<T>(0)))             \
  }                                                                                                \
  ROCSHMEM_API T rocshmem_##N##_atomic_fetch_add(T *dest, T value, int pe) {                       \
    return rocshmem_ctx_##N##_atomic_fetch_add(ROCSHMEM_CTX_DEFAULT, dest, value, pe);             \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_ctx_##N##_atomic_add(rocshmem_ctx_t ctx, T *dest, T value, int pe) {  \
    ROCSHMEM_AMO_DISPATCH_VOID(detail::amo_add<T>(dest, value, detail::ctx_pe(ctx, pe)),           \
                               ROCSHMEM_HOST_AMO(T, D, ROCSHMEM_AMO_ADD, dest, value, static_cast<T>(0)))        \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_##N##_atomic_add(T *dest, T value, int pe) {                          \
    rocshmem_ctx_##N##_atomic_add(ROCSHMEM_CTX_DEFAULT, dest, value, pe);                          \
  }                                                                                                \
  ROCSHMEM_API T rocshmem_ctx_##N##_atomic_fetch_inc(rocshmem_ctx_t ctx, T *dest, int pe) {        \
    return rocshmem_ctx_##N##_atomic_fetch_add(ctx, dest, static_cast<T>(1), pe);                               \
  }                                                                                                \
  ROCSHMEM_API T rocshmem_##N##_atomic_fetch_inc(T *dest, int pe) {                                \
    return rocshmem_ctx_##N##_atomic_fetch_add(ROCSHMEM_CTX_DEFAULT, dest, static_cast<T>(1), pe);              \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_ctx_##N##_atomic_inc(rocshmem_ctx_t ctx, T *dest, int pe) {           \
    rocshmem_ctx_##N##_atomic_add(ctx, dest, static_cast<T>(1), pe);                                            \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_##N##_atomic_inc(T *dest, int pe) {                                   \
    rocshmem_ctx_##N##_atomic_add(ROCSHMEM_CTX_DEFAULT, dest, static_cast<T>(1), pe);                           \
  }
ROCSHMEM_AMO_STANDARD_TYPES(ROCSHMEM_AMO_STANDARD)

#define ROCSHMEM_AMO_BITWISE_ONE(T, N, D, NAME, DEVFN, HOSTOP)                                     \
  ROCSHMEM_API T rocshmem_ctx_##N##_atomic_fetch_##NAME(rocshmem_ctx_t ctx, T *dest, T value, int pe) { \
    ROCSHMEM_AMO_DISPATCH(detail::DEVFN<T>(dest, value, detail::ctx_pe(ctx, pe)),                  \
                          ROCSHMEM_HOST_AMO(T, D, HOSTOP, dest, value, static_cast<T>(0)))                       \
  }                                                                                                \
  ROCSHMEM_API T rocshmem_##N##_atomic_fetch_##NAME(T *dest, T value, int pe) {                    \
    return rocshmem_ctx_##N##_atomic_fetch_##NAME(ROCSHMEM_CTX_DEFAULT, dest, value, pe);          \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_ctx_##N##_atomic_##NAME(rocshmem_ctx_t ctx, T *dest, T value, int pe) { \
    ROCSHMEM_AMO_DISPATCH_VOID(detail::DEVFN<T>(dest, value, detail::ctx_pe(ctx, pe)),             \
                               ROCSHMEM_HOST_AMO(T, D, HOSTOP, dest, value, static_cast<T>(0)))                  \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_##N##_atomic_##NAME(T *dest, T value, int pe) {                       \
    rocshmem_ctx_##N##_atomic_##NAME(ROCSHMEM_CTX_DEFAULT, dest, value, pe);                       \
  }
#define ROCSHMEM_AMO_BITWISE(T, N, D)                                                              \
  ROCSHMEM_AMO_BITWISE_ONE(T, N, D, and, amo_fetch_and, ROCSHMEM_AMO_AND)                          \
  ROCSHMEM_AMO_BITWISE_ONE(T, N, D, or, amo_fetch_or, ROCSHMEM_AMO_OR)                             \
  ROCSHMEM_AMO_BITWISE_ONE(T, N, D, xor, amo_fetch_xor, ROCSHMEM_AMO_XOR)
ROCSHMEM_AMO_BITWISE_TYPES(ROCSHMEM_AMO_BITWISE)

// ===================================================================================================
// Point-to-point synchronisation (host + device)
// ===================================================================================================

#if defined(__CUDA_ARCH__)
#define ROCSHMEM_SYNC_BODY(dev_stmt, host_stmt) dev_stmt
#else
#define ROCSHMEM_SYNC_BODY(dev_stmt, host_stmt) host_stmt
#endif

namespace api_detail {
// Host helper: converts typed operand arrays into the engine's bit arrays.
template <typename T>
struct HostOperands {
  uint64_t one;
  uint64_t *many;
  HostOperands(T v) : one(bits_of<T>(v)), many(nullptr) {}
  HostOperands(const T *vals, size_t n) : one(0), many(new uint64_t[n ? n : 1]) {
    for (size_t i = 0; i < n; ++i) many[i] = bits_of<T>(vals[i]);
  }
  ~HostOperands() { delete[] many; }
  const uint64_t *data() const { return many ? many : &one; }
};
}  // namespace api_detail

#define ROCSHMEM_SYNC_TYPED(T, N, D)                                                               \
  ROCSHMEM_API void rocshmem_##N##_wait_until(T *ivars, int cmp, T val) {                          \
    ROCSHMEM_SYNC_BODY(detail::stat_add(ROCSHMEM_STAT_WAIT); detail::wait_until<T>(ivars, cmp, val);, \
                       host::wait_until(ivars, D, cmp, api_detail::bits_of<T>(val));)              \
  }                                                                                                \
  ROCSHMEM_API int rocshmem_##N##_test(T *ivars, int cmp, T val) {                                 \
    ROCSHMEM_SYNC_BODY(detail::stat_add(ROCSHMEM_STAT_TEST); return detail::test<T>(ivars, cmp, val);, \
                       return host::test(ivars, D, cmp, api_detail::bits_of<T>(val));)             \
  }                                                                                                \
  /* Extension: ROCSHMEM_SUCCESS, or ROCSHMEM_ERROR when the wait budget ran out. */               \
  ROCSHMEM_API int rocshmemx_##N##_wait_until_status(T *ivars, int cmp, T val) {                   \
    ROCSHMEM_SYNC_BODY(return detail::wait_until<T>(ivars, cmp, val);,                             \
                       return host::wait_until(ivars, D, cmp, api_detail::bits_of<T>(val));)       \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_##N##_wait_until_all(T *ivars, size_t nelems, const int *status, int cmp, T val) { \
    ROCSHMEM_SYNC_BODY((detail::wait_until_all<T, false>(ivars, nelems, status, cmp, &val));,      \
                       { api_detail::HostOperands<T> o(val);                                       \
                         host::wait_until_all(ivars, nelems, status, D, cmp, o.data(), false); })  \
  }                                                                                                \
  ROCSHMEM_API size_t rocshmem_##N##_wait_until_any(T *ivars, size_t nelems, const int *status, int cmp, T val) { \
    ROCSHMEM_SYNC_BODY(return (detail::wait_until_any<T, false>(ivars, nelems, status, cmp, &val));, \
                       { api_detail::HostOperands<T> o(val);                                       \
                         return host::wait_until_any(ivars, nelems, status, D, cmp, o.data(), false); }) \
  }                                                                                                \
  ROCSHMEM_API size_t rocshmem_##N##_wait_until_some(T *ivars, size_t nelems, size_t *indices,     \
                                                     const int *status, int cmp, T val) {          \
    ROCSHMEM_SYNC_BODY(return (detail::wait_until_some<T, false>(ivars, nelems, indices, status, cmp, &val));, \
                       { api_detail::HostOperands<T> o(val);                                       \
                         return host::wait_until_some(ivars, nelems, indices, status, D, cmp, o.data(), false); }) \
  }                                                                                                \
  ROCSHMEM_API void rocshmem_##N##_wait_until_all_vector(T *ivars, size_t nelems, const int *status, \
                                                         int cmp, T *vals) {                       \
    ROCSHMEM_SYNC_BODY((detail::wait_until_all<T, true>(ivars, nelems, status, cmp, vals));,       \
                       { api_detail::HostOperands<T> o(vals, nelems);                              \
                         host::wait_until_all(ivars, nelems, status, D, cmp, o.data(), true); })   \
  }                                                                                                \
  ROCSHMEM_API size_t rocshmem_##N##_wait_until_any_vector(T *ivars, size_t nelems, const int *status, \
                                                           int cmp, T *vals) {                     \
    ROCSHMEM_SYNC_BODY(return (detail::wait_until_any<T, true>(ivars, nelems, status, cmp, vals));, \
                       { api_detail::HostOperands<T> o(vals, nelems);                              \
                         return host::wait_until_any(ivars, nelems, status, D, cmp, o.data(), true); }) \
  }                                                                                                \
  ROCSHMEM_API size_t rocshmem_##N##_wait_until_some_vector(T *ivars, size_t nelems, size_t *indices, \
                                                            const int *status, int cmp, T *vals) { \
    ROCSHMEM_SYNC_BODY(return (detail::wait_until_some<T, true>(ivars, nelems, indices, status, cmp, vals));, \
                       { api_detail::HostOperands<T> o(vals, nelems);                              \
                         return host::wait_until_some(ivars, nelems, indices, status, D, cmp, o.data(), true); }) \
  }
ROCSHMEM_SYNC_TYPES(ROCSHMEM_SYNC_TYPED)

// ===================================================================================================
// Host collectives
// ===================================================================================================

#define ROCSHMEM_HOST_COLL_TYPED(T, N)                                                             \
  inline void rocshmem_ctx_##N##_broadcast(rocshmem_ctx_t ctx, rocshmem_team_t team, T *dest,      \
                                           const T *source, int nelems, int pe_root) {             \
    host::broadcast(ctx, team, dest, source, size_t(nelems) * sizeof(T), pe_root);                 \
  }                                                                                                \
  inline void rocshmem_ctx_##N##_broadcast(rocshmem_ctx_t ctx, T *dest, const T *source, int nelems, \
                                           int pe_root, int pe_start, int log_pe_stride,           \
                                           int pe_size, long *) {                                  \
    host::broadcast_active_set(ctx, dest, source, size_t(nelems) * sizeof(T), pe_root, pe_start,   \
                               log_pe_stride, pe_size);                                            \
  }                                                                                                \
  inline void rocshmem_ctx_##N##_fcollect(rocshmem_ctx_t ctx, rocshmem_team_t team, T *dest,       \
                                          const T *source, int nelems) {                           \
    host::fcollect(ctx, team, dest, source, size_t(nelems) * sizeof(T));                           \
  }                                                                                                \
  inline void rocshmem_ctx_##N##_alltoall(rocshmem_ctx_t ctx, rocshmem_team_t team, T *dest,       \
                                          const T *source, int nelems) {                           \
    host::alltoall(ctx, team, dest, source, size_t(nelems) * sizeof(T));                           \
  }
ROCSHMEM_STANDARD_RMA_TYPES(ROCSHMEM_HOST_COLL_TYPED)

#define ROCSHMEM_HOST_REDUCE_ONE(T, N, D, OPNAME, OP)                                              \
  inline int rocshmem_ctx_##N##_##OPNAME##_reduce(rocshmem_ctx_t ctx, rocshmem_team_t team, T *dest, \
                                                  const T *source, int nreduce) {                  \
    return host::reduce(ctx, team, dest, source, size_t(nreduce), D, OP);                          \
  }                                                                                                \
  inline void rocshmem_ctx_##N##_##OPNAME##_to_all(rocshmem_ctx_t ctx, T *dest, const T *source,   \
                                                   int nreduce, int PE_start, int logPE_stride,    \
                                                   int PE_size, T *, long *) {                     \
    host::reduce_active_set(ctx, dest, source, size_t(nreduce), D, OP, PE_start, logPE_stride, PE_size); \
  }
#define ROCSHMEM_HOST_REDUCE_ARITH(T, N, D)                                                        \
  ROCSHMEM_HOST_REDUCE_ONE(T, N, D, sum, ROCSHMEM_SUM)                                             \
  ROCSHMEM_HOST_REDUCE_ONE(T, N, D, min, ROCSHMEM_MIN)                                             \
  ROCSHMEM_HOST_REDUCE_ONE(T, N, D, max, ROCSHMEM_MAX)                                             \
  ROCSHMEM_HOST_REDUCE_ONE(T, N, D, prod, ROCSHMEM_PROD)
#define ROCSHMEM_HOST_REDUCE_BITWISE(T, N, D)                                                      \
  ROCSHMEM_HOST_REDUCE_ONE(T, N, D, or, ROCSHMEM_OR)                                               \
  ROCSHMEM_HOST_REDUCE_ONE(T, N, D, and, ROCSHMEM_AND)                                             \
  ROCSHMEM_HOST_REDUCE_ONE(T, N, D, xor, ROCSHMEM_XOR)
ROCSHMEM_REDUCE_INT_TYPES(ROCSHMEM_HOST_REDUCE_ARITH)
ROCSHMEM_REDUCE_INT_TYPES(ROCSHMEM_HOST_REDUCE_BITWISE)
ROCSHMEM_REDUCE_FLOAT_TYPES(ROCSHMEM_HOST_REDUCE_ARITH)

}  // namespace rocshmem

#if defined(__CUDACC__)
#include "rocshmem_device_api.cuh"
#endif
