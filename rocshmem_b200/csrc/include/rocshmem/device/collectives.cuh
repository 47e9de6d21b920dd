// Block-collective device routines: contexts, teams, barrier / sync, broadcast, fcollect, alltoall
// and reductions, callable from inside user kernels by all threads of one block.
//
// Reference counterparts: internal_direct_barrier / internal_atomic_barrier / barrier_all / sync
// (src/ipc/context_ipc_device_coll.cpp:31-123), internal_direct_allreduce / internal_ring_allreduce
// (src/ipc/context_ipc_tmpl_device.hpp:166-417), broadcast / alltoall_linear / fcollect_linear
// (:420-531), wg_ctx_create (src/rocshmem_gpu.cpp:286-325). Design differences:
//   * Barrier: every member writes its team epoch into its own slot on every member (one hop
//     through NVSwitch, all peers in parallel, one thread per peer) and waits until all slots of its
//     own array have reached that epoch. Epochs only grow, so there is no reset phase and no
//     root; the reference funnels 2(n-1) messages through a root in two hops and resets pSync.
//   * Reduction: one bandwidth-optimal algorithm for every size. Each member reduces "its" slice by
//     loading that slice from every member's source (symmetric, so no staging buffer) and stores the
//     result into every member's dest. Per member, (n-1)/n of the payload is read and written over
//     NVLink, dest == source is safe, and there is no 1024-element work buffer that forces the
//     reference into many small ring steps.
//   * Collectives on one team share the team's barrier flags, so, as in the reference, two
//     collectives on the same team must not run concurrently (one block per team at a time).
#pragma once

#include "primitives.cuh"

namespace rocshmem {
namespace detail {

// ---- teams and contexts ----------------------------------------------------------------------------

__device__ __forceinline__ rocshmem_team_dev *team_of(rocshmem_team_t team) {
  // Handles are addresses on the process's first PE; rebase to the block's own PE.
  return local_ptr(team);
}
__device__ __forceinline__ rocshmem_team_dev *world_team() { return st().teams; }

__device__ __forceinline__ rocshmem_team_dev *ctx_team(const rocshmem_ctx_t &ctx) {
  if (ctx.team_opaque == nullptr) return world_team();
  return local_ptr(static_cast<rocshmem_team_dev *>(ctx.team_opaque));
}

// Team-relative PE -> world PE for operations issued through a context.
__device__ __forceinline__ int ctx_pe(const rocshmem_ctx_t &ctx, int pe) {
  if (ctx.team_opaque == nullptr) return pe;
  const rocshmem_team_dev *t = ctx_team(ctx);
  return t->pe_start + pe * t->stride;
}

__device__ __forceinline__ long long ctx_options(const rocshmem_ctx_t &ctx) {
  if (ctx.ctx_opaque == nullptr) return 0;
  return local_ptr(static_cast<rocshmem_ctx_dev *>(ctx.ctx_opaque))->options;
}

__device__ __forceinline__ int team_pe_to_world(const rocshmem_team_dev *t, int pe) {
  return t->pe_start + pe * t->stride;
}

__device__ __forceinline__ int team_translate(rocshmem_team_t src, int src_pe, rocshmem_team_t dst) {
  if (src == nullptr || dst == nullptr) return -1;
  const rocshmem_team_dev *s = team_of(src), *d = team_of(dst);
  if (src_pe < 0 || src_pe >= s->size) return -1;
  int w = s->pe_start + src_pe * s->stride;
  if (w < d->pe_start) return -1;
  int off = w - d->pe_start;
  if (off % d->stride) return -1;
  int idx = off / d->stride;
  return idx < d->size ? idx : -1;
}

// Takes a context from the pool (bitmask, lock-free). Block-collective: thread 0 allocates and the
// handle is written to *ctx, which normally lives in shared memory.
__device__ inline int ctx_create(long long options, rocshmem_team_dev *team, rocshmem_ctx_t *ctx) {
  int rc = 0;
  if (block_tid() == 0) {
    const rocshmem_device_state &s = st();
    int found = -1;
    const int words = (s.max_ctxs + 63) / 64;
    for (int w = 0; w < words && found < 0; ++w) {
      unsigned long long m = s.ctx_free_mask[w];
      while (m != 0) {
        int bit = __ffsll(static_cast<long long>(m)) - 1;
        unsigned long long old = atomicAnd(&s.ctx_free_mask[w], ~(1ull << bit));
        if (old & (1ull << bit)) {
          found = w * 64 + bit;
          break;
        }
        m = old & ~(1ull << bit);
      }
    }
    if (found < 0) {
      ctx->ctx_opaque = nullptr;
      ctx->team_opaque = nullptr;
      rc = -1;
    } else {
      rocshmem_ctx_dev *c = &s.ctxs[found];
      c->options = options;
      c->team = team;
      c->id = found;
      c->in_use = 1;
      c->ops = 0;
      // Handles are expressed relative to the process's first PE, like every other handle.
      char *rebased = reinterpret_cast<char *>(c) - size_t(s.local_index) * s.heap_stride;
      ctx->ctx_opaque = rebased;
      ctx->team_opaque = reinterpret_cast<char *>(team) - size_t(s.local_index) * s.heap_stride;
      stat_add(ROCSHMEM_STAT_CTX_CREATE);
    }
  }
  __syncthreads();
  // All threads return the same code: thread 0's result is read back from the handle.
  if (block_tid() != 0) rc = (ctx->ctx_opaque == nullptr) ? -1 : 0;
  return rc;
}

__device__ inline void ctx_destroy(rocshmem_ctx_t *ctx) {
  __syncthreads();
  if (block_tid() == 0 && ctx->ctx_opaque != nullptr) {
    const rocshmem_device_state &s = st();
    rocshmem_ctx_dev *c = local_ptr(static_cast<rocshmem_ctx_dev *>(ctx->ctx_opaque));
    int id = c->id;
    c->in_use = 0;
    __threadfence();
    atomicOr(&s.ctx_free_mask[id / 64], 1ull << (id % 64));
    ctx->ctx_opaque = nullptr;
    stat_add(ROCSHMEM_STAT_CTX_DESTROY);
  }
  __syncthreads();
}

// ---- collectives through the host proxy ------------------------------------------------------------------

// With bit 2 of use_proxy set, a block-level collective is one blocking command: thread 0 submits it, the host
// thread runs the host form of the collective for the team, the block waits (reference: ROContext's
// collectives, src/reverse_offload/context_ro_tmpl_device.hpp:111-374). Needs one PE per process: the host
// form acts for all PEs of its process at once.
__device__ __forceinline__ bool proxy_collectives_on() { return (st().use_proxy & 4) != 0; }

// Element type codes of the host engine (rocshmem_dtype in rocshmem_host.h).
template <typename T> struct ProxyDtype;
template <> struct ProxyDtype<signed char> { static constexpr int code = 0; };
template <> struct ProxyDtype<char> { static constexpr int code = 0; };
template <> struct ProxyDtype<unsigned char> { static constexpr int code = 1; };
template <> struct ProxyDtype<short> { static constexpr int code = 2; };
template <> struct ProxyDtype<unsigned short> { static constexpr int code = 3; };
template <> struct ProxyDtype<int> { static constexpr int code = 4; };
template <> struct ProxyDtype<unsigned int> { static constexpr int code = 5; };
template <> struct ProxyDtype<long> { static constexpr int code = 6; };
template <> struct ProxyDtype<long long> { static constexpr int code = 6; };
template <> struct ProxyDtype<unsigned long> { static constexpr int code = 7; };
template <> struct ProxyDtype<unsigned long long> { static constexpr int code = 7; };
template <> struct ProxyDtype<float> { static constexpr int code = 8; };
template <> struct ProxyDtype<double> { static constexpr int code = 9; };
template <> struct ProxyDtype<__half> { static constexpr int code = 10; };
template <> struct ProxyDtype<__nv_bfloat16> { static constexpr int code = 11; };

// Block-collective. `pe` carries the root of a broadcast, `cond` the element type of a reduction.
__device__ inline int proxy_collective(unsigned type, const rocshmem_team_dev *t, void *dest, const void *source,
                                       unsigned long long size, int pe, unsigned long long cond, unsigned op) {
  __shared__ int proxy_collective_rc;
  __syncthreads();   // the block's earlier writes (and a previous call's result) are settled
  if (block_tid() == 0) {
    bool ok = false;
    __threadfence_system();
    unsigned long long status = proxy_submit(type, pe, dest, source, size, cond, op, 1, true, &ok,
                                             static_cast<unsigned long long>(t->slot));
    proxy_collective_rc = (ok && status == 0) ? ROCSHMEM_SUCCESS : ROCSHMEM_ERROR;
  }
  __syncthreads();
  return proxy_collective_rc;
}

// ---- barrier ------------------------------------------------------------------------------------------

// Block-collective. Returns ROCSHMEM_SUCCESS or ROCSHMEM_ERROR (a peer did not arrive in time).
// `through_proxy` == false is for the library's own barrier kernel: it is what the host (and the proxy thread, for
// a proxied barrier) launches, so it must signal over NVLink itself instead of asking the proxy again.
__device__ inline int team_barrier(rocshmem_team_dev *t, bool through_proxy = true) {
  const rocshmem_device_state &s = st();
  const unsigned tid = block_tid(), nthr = block_threads();
  if (t->my_pe < 0) return ROCSHMEM_ERROR;
  if (through_proxy && proxy_collectives_on()) {
    return proxy_collective(ROCSHMEM_PROXY_BARRIER, t, nullptr, nullptr, 0, 0, 0, 0);
  }
  __syncthreads();  // everything the block did before the barrier is ordered before the signals
  if (tid == 0) t->barrier_epoch = t->barrier_epoch + 1;
  __syncthreads();
  const unsigned long long epoch = *reinterpret_cast<volatile unsigned long long *>(&t->barrier_epoch);
  unsigned long long *mine = s.barrier_flags + size_t(t->slot) * ROCSHMEM_MAX_PES;
  for (unsigned j = tid; j < static_cast<unsigned>(t->size); j += nthr) {
    int w = team_pe_to_world(t, static_cast<int>(j));
    // Release at system scope: cumulative over the block's earlier writes (ordered by the barrier
    // above), so a peer that acquires this flag sees them.
    st_release_sys(remote_ptr(mine + t->my_pe, w), epoch);
  }
  bool ok = true;
  for (unsigned j = tid; j < static_cast<unsigned>(t->size); j += nthr) {
    ok = wait_ge_sys(mine + j, epoch, team_pe_to_world(t, static_cast<int>(j)), 50,
                     ROCSHMEM_ERR_BARRIER_TIMEOUT) && ok;
  }
  int all_ok = __syncthreads_and(ok ? 1 : 0);
  return all_ok ? ROCSHMEM_SUCCESS : ROCSHMEM_ERROR;
}

// ---- reduction helpers -----------------------------------------------------------------------------------

template <typename T, int OP>
__device__ __forceinline__ T reduce_op(T a, T b) {
  if (OP == ROCSHMEM_SUM) return a + b;
  if (OP == ROCSHMEM_PROD) return a * b;
  if (OP == ROCSHMEM_MIN) return a < b ? a : b;
  if (OP == ROCSHMEM_MAX) return a > b ? a : b;
  return b;
}
template <typename T, int OP>
__device__ __forceinline__ T reduce_bitop(T a, T b) {
  if (OP == ROCSHMEM_AND) return a & b;
  if (OP == ROCSHMEM_OR) return a | b;
  if (OP == ROCSHMEM_XOR) return a ^ b;
  return reduce_op<T, OP>(a, b);
}

// Accumulation type: 16-bit floating types are summed in fp32.
template <typename T> struct Acc { using type = T; };
template <> struct Acc<__half> { using type = float; };
template <> struct Acc<__nv_bfloat16> { using type = float; };

template <typename T> __device__ __forceinline__ typename Acc<T>::type to_acc(T v) { return v; }
template <> __device__ __forceinline__ float to_acc<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_acc<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_acc(typename Acc<T>::type v) { return v; }
template <> __device__ __forceinline__ __half from_acc<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T, int OP, bool BITWISE>
__device__ __forceinline__ typename Acc<T>::type apply(typename Acc<T>::type a, typename Acc<T>::type b) {
  if constexpr (BITWISE) {
    return reduce_bitop<typename Acc<T>::type, OP>(a, b);
  } else {
    return reduce_op<typename Acc<T>::type, OP>(a, b);
  }
}

// Reduce elements [lo, hi) of `source` over all members and store the result into every member's
// `dest`. Vector path: 16 bytes per thread per member when all bases are 16-byte aligned.
template <typename T, int OP, bool BITWISE>
__device__ inline void reduce_slice(rocshmem_team_dev *t, T *dest, const T *source, size_t lo,
                                    size_t hi, unsigned tid, unsigned nthr) {
  using A = typename Acc<T>::type;
  constexpr int VEC = 16 / sizeof(T);
  const int n = t->size;
  const bool aligned = ((reinterpret_cast<uintptr_t>(dest) | reinterpret_cast<uintptr_t>(source)) & 15u) == 0 &&
                       (lo % VEC) == 0;
  size_t i = lo;
  if (aligned) {
    const size_t nvec = (hi - lo) / VEC;
    for (size_t v = tid; v < nvec; v += nthr) {
      const size_t e = lo + v * VEC;
      A acc[VEC];
      {
        int4 raw = *reinterpret_cast<const int4 *>(remote_ptr(source + e, team_pe_to_world(t, 0)));
        const T *x = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] = to_acc<T>(x[k]);
      }
      for (int j = 1; j < n; ++j) {
        int4 raw = *reinterpret_cast<const int4 *>(remote_ptr(source + e, team_pe_to_world(t, j)));
        const T *x = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] = apply<T, OP, BITWISE>(acc[k], to_acc<T>(x[k]));
      }
      int4 out;
      T *o = reinterpret_cast<T *>(&out);
#pragma unroll
      for (int k = 0; k < VEC; ++k) o[k] = from_acc<T>(acc[k]);
      for (int j = 0; j < n; ++j) {
        *reinterpret_cast<int4 *>(remote_ptr(dest + e, team_pe_to_world(t, j))) = out;
      }
    }
    i = lo + nvec * VEC;
  }
  for (size_t e = i + tid; e < hi; e += nthr) {
    A acc = to_acc<T>(*remote_ptr(source + e, team_pe_to_world(t, 0)));
    for (int j = 1; j < n; ++j) {
      acc = apply<T, OP, BITWISE>(acc, to_acc<T>(*remote_ptr(source + e, team_pe_to_world(t, j))));
    }
    T out = from_acc<T>(acc);
    for (int j = 0; j < n; ++j) *remote_ptr(dest + e, team_pe_to_world(t, j)) = out;
  }
}

template <typename T, int OP, bool BITWISE>
__device__ inline int team_reduce(rocshmem_team_dev *t, T *dest, const T *source, size_t nreduce) {
  if (nreduce == 0) return ROCSHMEM_SUCCESS;
  if (t->my_pe < 0) return ROCSHMEM_ERROR;
  stat_add(ROCSHMEM_STAT_REDUCE);
  if (proxy_collectives_on()) {
    return proxy_collective(ROCSHMEM_PROXY_REDUCE, t, dest, source, nreduce, 0, ProxyDtype<T>::code, OP);
  }
  // Sources of all members are complete.
  if (team_barrier(t) != ROCSHMEM_SUCCESS) return ROCSHMEM_ERROR;
  constexpr size_t VEC = 16 / sizeof(T);
  const size_t n = static_cast<size_t>(t->size);
  // Slices are multiples of one 16-byte vector so that the vector path applies to each of them.
  size_t per = ((nreduce + n - 1) / n + VEC - 1) / VEC * VEC;
  size_t lo = per * static_cast<size_t>(t->my_pe);
  size_t hi = lo + per;
  if (lo > nreduce) lo = nreduce;
  if (hi > nreduce) hi = nreduce;
  reduce_slice<T, OP, BITWISE>(t, dest, source, lo, hi, block_tid(), block_threads());
  // All slices have landed everywhere; sources may be reused.
  return team_barrier(t);
}

// ---- broadcast / fcollect / alltoall ----------------------------------------------------------------------

// The root stores into every other member's dest (its own dest is left untouched, as in the
// reference), then the team synchronises.
__device__ inline void team_broadcast(rocshmem_team_dev *t, void *dest, const void *source,
                                      size_t bytes, int pe_root) {
  if (bytes == 0 || t->my_pe < 0) return;
  stat_add(ROCSHMEM_STAT_BROADCAST);
  if (proxy_collectives_on()) {
    proxy_collective(ROCSHMEM_PROXY_BROADCAST, t, dest, source, bytes, pe_root, 0, 0);
    return;
  }
  if (t->my_pe == pe_root) {
    Group<Scope::BLOCK> g;
    for (int j = 0; j < t->size; ++j) {
      if (j == pe_root) continue;
      copy_bytes<Scope::BLOCK>(remote_ptr(static_cast<char *>(dest), team_pe_to_world(t, j)), source,
                               bytes, g);
    }
  }
  team_barrier(t);
}

// dest[my_pe * bytes ...) on every member receives my source.
__device__ inline void team_fcollect(rocshmem_team_dev *t, void *dest, const void *source, size_t bytes) {
  if (bytes == 0 || t->my_pe < 0) return;
  stat_add(ROCSHMEM_STAT_FCOLLECT);
  if (proxy_collectives_on()) {
    proxy_collective(ROCSHMEM_PROXY_FCOLLECT, t, dest, const_cast<void *>(source), bytes, 0, 0, 0);
    return;
  }
  Group<Scope::BLOCK> g;
  char *slot = static_cast<char *>(dest) + size_t(t->my_pe) * bytes;
  for (int d = 0; d < t->size; ++d) {
    int j = (t->my_pe + d) % t->size;  // start with myself, then rotate so peers are hit evenly
    copy_bytes<Scope::BLOCK>(remote_ptr(slot, team_pe_to_world(t, j)), source, bytes, g);
  }
  team_barrier(t);
}

// Member i sends source[j * bytes ...) to member j, which stores it at dest[i * bytes ...).
__device__ inline void team_alltoall(rocshmem_team_dev *t, void *dest, const void *source, size_t bytes) {
  if (bytes == 0 || t->my_pe < 0) return;
  stat_add(ROCSHMEM_STAT_ALLTOALL);
  if (proxy_collectives_on()) {
    proxy_collective(ROCSHMEM_PROXY_ALLTOALL, t, dest, const_cast<void *>(source), bytes, 0, 0, 0);
    return;
  }
  Group<Scope::BLOCK> g;
  char *slot = static_cast<char *>(dest) + size_t(t->my_pe) * bytes;
  for (int d = 0; d < t->size; ++d) {
    int j = (t->my_pe + d) % t->size;
    copy_bytes<Scope::BLOCK>(remote_ptr(slot, team_pe_to_world(t, j)),
                             static_cast<const char *>(source) + size_t(j) * bytes, bytes, g);
  }
  team_barrier(t);
}

}  // namespace detail
}  // namespace rocshmem
