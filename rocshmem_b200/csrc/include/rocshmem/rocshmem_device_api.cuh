// Device-only API families: warp / block RMA, put-with-signal, block collectives.
// Included at the end of rocshmem.h when compiling with nvcc.
//
// Reference counterparts: include/rocshmem/rocshmem_RMA_X.hpp (wave / wg put, get and their nbi
// forms), rocshmem_SIG_OP.hpp (put_signal in six granularities, signal_fetch in three) and the
// device half of rocshmem_COLL.hpp (wg_alltoall, wg_broadcast, wg_fcollect, wg_reduce). Every
// function exists under its _warp / _block name and under the reference's _wave / _wg alias.
#pragma once

namespace rocshmem {

// ---- warp / block RMA ----------------------------------------------------------------------------------

#define ROCSHMEM_X_MEM(SUF, SCOPE, STAT)                                                           \
  ROCSHMEM_DEVICE_API void rocshmem_ctx_putmem_##SUF(rocshmem_ctx_t ctx, void *dest, const void *source, size_t nelems, int pe) { \
    detail::stat_add(STAT);                                                                        \
    detail::putmem<detail::Scope::SCOPE>(dest, source, nelems, detail::ctx_pe(ctx, pe), true, !ROCSHMEM_DEV_NOSTORE(ctx)); \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_putmem_##SUF(void *dest, const void *source, size_t nelems, int pe) { \
    rocshmem_ctx_putmem_##SUF(ROCSHMEM_CTX_DEFAULT, dest, source, nelems, pe);                     \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_ctx_putmem_nbi_##SUF(rocshmem_ctx_t ctx, void *dest, const void *source, size_t nelems, int pe) { \
    detail::stat_add(STAT);                                                                        \
    detail::putmem<detail::Scope::SCOPE>(dest, source, nelems, detail::ctx_pe(ctx, pe), false, false); \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_putmem_nbi_##SUF(void *dest, const void *source, size_t nelems, int pe) { \
    rocshmem_ctx_putmem_nbi_##SUF(ROCSHMEM_CTX_DEFAULT, dest, source, nelems, pe);                 \
  }
#define ROCSHMEM_X_GETMEM(SUF, SCOPE, STAT)                                                        \
  ROCSHMEM_DEVICE_API void rocshmem_ctx_getmem_##SUF(rocshmem_ctx_t ctx, void *dest, const void *source, size_t nelems, int pe) { \
    detail::stat_add(STAT);                                                                        \
    detail::getmem<detail::Scope::SCOPE>(dest, source, nelems, detail::ctx_pe(ctx, pe), true);     \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_getmem_##SUF(void *dest, const void *source, size_t nelems, int pe) { \
    rocshmem_ctx_getmem_##SUF(ROCSHMEM_CTX_DEFAULT, dest, source, nelems, pe);                     \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_ctx_getmem_nbi_##SUF(rocshmem_ctx_t ctx, void *dest, const void *source, size_t nelems, int pe) { \
    detail::stat_add(STAT);                                                                        \
    detail::getmem<detail::Scope::SCOPE>(dest, source, nelems, detail::ctx_pe(ctx, pe), false);    \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_getmem_nbi_##SUF(void *dest, const void *source, size_t nelems, int pe) { \
    rocshmem_ctx_getmem_nbi_##SUF(ROCSHMEM_CTX_DEFAULT, dest, source, nelems, pe);                 \
  }
ROCSHMEM_X_MEM(warp, WARP, ROCSHMEM_STAT_PUT_WARP)
ROCSHMEM_X_MEM(wave, WARP, ROCSHMEM_STAT_PUT_WARP)
ROCSHMEM_X_MEM(block, BLOCK, ROCSHMEM_STAT_PUT_BLOCK)
ROCSHMEM_X_MEM(wg, BLOCK, ROCSHMEM_STAT_PUT_BLOCK)
ROCSHMEM_X_GETMEM(warp, WARP, ROCSHMEM_STAT_GET_WARP)
ROCSHMEM_X_GETMEM(wave, WARP, ROCSHMEM_STAT_GET_WARP)
ROCSHMEM_X_GETMEM(block, BLOCK, ROCSHMEM_STAT_GET_BLOCK)
ROCSHMEM_X_GETMEM(wg, BLOCK, ROCSHMEM_STAT_GET_BLOCK)

#define ROCSHMEM_X_TYPED_ONE(T, N, SUF)                                                            \
  ROCSHMEM_DEVICE_API void rocshmem_ctx_##N##_put_##SUF(rocshmem_ctx_t ctx, T *dest, const T *source, size_t nelems, int pe) { \
    rocshmem_ctx_putmem_##SUF(ctx, dest, source, nelems * sizeof(T), pe);                          \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_##N##_put_##SUF(T *dest, const T *source, size_t nelems, int pe) { \
    rocshmem_ctx_putmem_##SUF(ROCSHMEM_CTX_DEFAULT, dest, source, nelems * sizeof(T), pe);         \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_ctx_##N##_put_nbi_##SUF(rocshmem_ctx_t ctx, T *dest, const T *source, size_t nelems, int pe) { \
    rocshmem_ctx_putmem_nbi_##SUF(ctx, dest, source, nelems * sizeof(T), pe);                      \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_##N##_put_nbi_##SUF(T *dest, const T *source, size_t nelems, int pe) { \
    rocshmem_ctx_putmem_nbi_##SUF(ROCSHMEM_CTX_DEFAULT, dest, source, nelems * sizeof(T), pe);     \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_ctx_##N##_get_##SUF(rocshmem_ctx_t ctx, T *dest, const T *source, size_t nelems, int pe) { \
    rocshmem_ctx_getmem_##SUF(ctx, dest, source, nelems * sizeof(T), pe);                          \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_##N##_get_##SUF(T *dest, const T *source, size_t nelems, int pe) { \
    rocshmem_ctx_getmem_##SUF(ROCSHMEM_CTX_DEFAULT, dest, source, nelems * sizeof(T), pe);         \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_ctx_##N##_get_nbi_##SUF(rocshmem_ctx_t ctx, T *dest, const T *source, size_t nelems, int pe) { \
    rocshmem_ctx_getmem_nbi_##SUF(ctx, dest, source, nelems * sizeof(T), pe);                      \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_##N##_get_nbi_##SUF(T *dest, const T *source, size_t nelems, int pe) { \
    rocshmem_ctx_getmem_nbi_##SUF(ROCSHMEM_CTX_DEFAULT, dest, source, nelems * sizeof(T), pe);     \
  }
#define ROCSHMEM_X_TYPED(T, N)                                                                     \
  ROCSHMEM_X_TYPED_ONE(T, N, warp) ROCSHMEM_X_TYPED_ONE(T, N, wave)                                \
  ROCSHMEM_X_TYPED_ONE(T, N, block) ROCSHMEM_X_TYPED_ONE(T, N, wg)
ROCSHMEM_RMA_TYPES(ROCSHMEM_X_TYPED)

// ---- put with signal ---------------------------------------------------------------------------------------
// The non-blocking forms complete locally at once, so they share the blocking implementation (the
// payload has been read when the call returns; remote visibility follows the signal).

#define ROCSHMEM_SIG_MEM(SUF, SCOPE)                                                               \
  ROCSHMEM_DEVICE_API void rocshmem_ctx_putmem_signal##SUF(rocshmem_ctx_t ctx, void *dest, const void *source, \
                                                           size_t nelems, uint64_t *sig_addr, uint64_t signal, \
                                                           int sig_op, int pe) {                   \
    detail::stat_add(ROCSHMEM_STAT_PUT_SIGNAL);                                                    \
    detail::putmem_signal<detail::Scope::SCOPE>(dest, source, nelems, sig_addr, signal, sig_op,    \
                                                detail::ctx_pe(ctx, pe));                          \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_putmem_signal##SUF(void *dest, const void *source, size_t nelems, \
                                                       uint64_t *sig_addr, uint64_t signal, int sig_op, int pe) { \
    rocshmem_ctx_putmem_signal##SUF(ROCSHMEM_CTX_DEFAULT, dest, source, nelems, sig_addr, signal, sig_op, pe); \
  }
ROCSHMEM_SIG_MEM(, THREAD)
ROCSHMEM_SIG_MEM(_warp, WARP)
ROCSHMEM_SIG_MEM(_wave, WARP)
ROCSHMEM_SIG_MEM(_block, BLOCK)
ROCSHMEM_SIG_MEM(_wg, BLOCK)
ROCSHMEM_SIG_MEM(_nbi, THREAD)
ROCSHMEM_SIG_MEM(_nbi_warp, WARP)
ROCSHMEM_SIG_MEM(_nbi_wave, WARP)
ROCSHMEM_SIG_MEM(_nbi_block, BLOCK)
ROCSHMEM_SIG_MEM(_nbi_wg, BLOCK)

#define ROCSHMEM_SIG_TYPED_ONE(T, N, SUF)                                                          \
  ROCSHMEM_DEVICE_API void rocshmem_ctx_##N##_put_signal##SUF(rocshmem_ctx_t ctx, T *dest, const T *source, \
                                                              size_t nelems, uint64_t *sig_addr,   \
                                                              uint64_t signal, int sig_op, int pe) { \
    rocshmem_ctx_putmem_signal##SUF(ctx, dest, source, nelems * sizeof(T), sig_addr, signal, sig_op, pe); \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_##N##_put_signal##SUF(T *dest, const T *source, size_t nelems, \
                                                          uint64_t *sig_addr, uint64_t signal, int sig_op, int pe) { \
    rocshmem_ctx_putmem_signal##SUF(ROCSHMEM_CTX_DEFAULT, dest, source, nelems * sizeof(T), sig_addr, signal, sig_op, pe); \
  }
#define ROCSHMEM_SIG_TYPED(T, N)                                                                   \
  ROCSHMEM_SIG_TYPED_ONE(T, N, ) ROCSHMEM_SIG_TYPED_ONE(T, N, _warp) ROCSHMEM_SIG_TYPED_ONE(T, N, _wave) \
  ROCSHMEM_SIG_TYPED_ONE(T, N, _block) ROCSHMEM_SIG_TYPED_ONE(T, N, _wg)                           \
  ROCSHMEM_SIG_TYPED_ONE(T, N, _nbi) ROCSHMEM_SIG_TYPED_ONE(T, N, _nbi_warp)                       \
  ROCSHMEM_SIG_TYPED_ONE(T, N, _nbi_wave) ROCSHMEM_SIG_TYPED_ONE(T, N, _nbi_block)                 \
  ROCSHMEM_SIG_TYPED_ONE(T, N, _nbi_wg)
ROCSHMEM_STANDARD_RMA_TYPES(ROCSHMEM_SIG_TYPED)

ROCSHMEM_DEVICE_API uint64_t rocshmem_signal_fetch(const uint64_t *sig_addr) {
  detail::stat_add(ROCSHMEM_STAT_SIGNAL_FETCH);
  return detail::signal_fetch<detail::Scope::THREAD>(sig_addr);
}
ROCSHMEM_DEVICE_API uint64_t rocshmem_signal_fetch_warp(const uint64_t *sig_addr) {
  return detail::signal_fetch<detail::Scope::WARP>(sig_addr);
}
ROCSHMEM_DEVICE_API uint64_t rocshmem_signal_fetch_block(const uint64_t *sig_addr) {
  return detail::signal_fetch<detail::Scope::BLOCK>(sig_addr);
}
ROCSHMEM_DEVICE_API uint64_t rocshmem_signal_fetch_wave(const uint64_t *sig_addr) { return rocshmem_signal_fetch_warp(sig_addr); }
ROCSHMEM_DEVICE_API uint64_t rocshmem_signal_fetch_wg(const uint64_t *sig_addr) { return rocshmem_signal_fetch_block(sig_addr); }

// ---- block collectives -----------------------------------------------------------------------------------------

#define ROCSHMEM_COLL_TYPED_ONE(T, N, G)                                                           \
  ROCSHMEM_DEVICE_API void rocshmem_ctx_##N##_##G##_alltoall(rocshmem_ctx_t, rocshmem_team_t team, T *dest, \
                                                             const T *source, int nelems) {        \
    if (team == nullptr || nelems <= 0) return;                                                    \
    detail::team_alltoall(detail::team_of(team), dest, source, size_t(nelems) * sizeof(T));        \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_ctx_##N##_##G##_broadcast(rocshmem_ctx_t, rocshmem_team_t team, T *dest, \
                                                              const T *source, int nelems, int pe_root) { \
    if (team == nullptr || nelems <= 0) return;                                                    \
    detail::team_broadcast(detail::team_of(team), dest, source, size_t(nelems) * sizeof(T), pe_root); \
  }                                                                                                \
  ROCSHMEM_DEVICE_API void rocshmem_ctx_##N##_##G##_fcollect(rocshmem_ctx_t, rocshmem_team_t team, T *dest, \
                                                             const T *source, int nelems) {        \
    if (team == nullptr || nelems <= 0) return;                                                    \
    detail::team_fcollect(detail::team_of(team), dest, source, size_t(nelems) * sizeof(T));        \
  }
#define ROCSHMEM_COLL_TYPED(T, N) ROCSHMEM_COLL_TYPED_ONE(T, N, block) ROCSHMEM_COLL_TYPED_ONE(T, N, wg)
ROCSHMEM_STANDARD_RMA_TYPES(ROCSHMEM_COLL_TYPED)

#define ROCSHMEM_DEV_REDUCE_ONE(T, N, OPNAME, OP, BITWISE, G)                                      \
  ROCSHMEM_DEVICE_API int rocshmem_ctx_##N##_##OPNAME##_##G##_reduce(rocshmem_ctx_t, rocshmem_team_t team, \
                                                                     T *dest, const T *source, int nreduce) { \
    if (team == nullptr) return ROCSHMEM_ERROR;                                                    \
    if (nreduce <= 0) return ROCSHMEM_SUCCESS;                                                     \
    return detail::team_reduce<T, OP, BITWISE>(detail::team_of(team), dest, source, size_t(nreduce)); \
  }
#define ROCSHMEM_DEV_REDUCE_ARITH(T, N, D)                                                         \
  ROCSHMEM_DEV_REDUCE_ONE(T, N, sum, ROCSHMEM_SUM, false, block) ROCSHMEM_DEV_REDUCE_ONE(T, N, sum, ROCSHMEM_SUM, false, wg) \
  ROCSHMEM_DEV_REDUCE_ONE(T, N, min, ROCSHMEM_MIN, false, block) ROCSHMEM_DEV_REDUCE_ONE(T, N, min, ROCSHMEM_MIN, false, wg) \
  ROCSHMEM_DEV_REDUCE_ONE(T, N, max, ROCSHMEM_MAX, false, block) ROCSHMEM_DEV_REDUCE_ONE(T, N, max, ROCSHMEM_MAX, false, wg) \
  ROCSHMEM_DEV_REDUCE_ONE(T, N, prod, ROCSHMEM_PROD, false, block) ROCSHMEM_DEV_REDUCE_ONE(T, N, prod, ROCSHMEM_PROD, false, wg)
#define ROCSHMEM_DEV_REDUCE_BITWISE(T, N, D)                                                       \
  ROCSHMEM_DEV_REDUCE_ONE(T, N, or, ROCSHMEM_OR, true, block) ROCSHMEM_DEV_REDUCE_ONE(T, N, or, ROCSHMEM_OR, true, wg) \
  ROCSHMEM_DEV_REDUCE_ONE(T, N, and, ROCSHMEM_AND, true, block) ROCSHMEM_DEV_REDUCE_ONE(T, N, and, ROCSHMEM_AND, true, wg) \
  ROCSHMEM_DEV_REDUCE_ONE(T, N, xor, ROCSHMEM_XOR, true, block) ROCSHMEM_DEV_REDUCE_ONE(T, N, xor, ROCSHMEM_XOR, true, wg)
ROCSHMEM_REDUCE_INT_TYPES(ROCSHMEM_DEV_REDUCE_ARITH)
ROCSHMEM_REDUCE_INT_TYPES(ROCSHMEM_DEV_REDUCE_BITWISE)
ROCSHMEM_REDUCE_FLOAT_TYPES(ROCSHMEM_DEV_REDUCE_ARITH)
// 16-bit floating types (extension; sums are accumulated in fp32).
ROCSHMEM_DEV_REDUCE_ARITH(__half, half, 0)
ROCSHMEM_DEV_REDUCE_ARITH(__nv_bfloat16, bfloat16, 0)

}  // namespace rocshmem
