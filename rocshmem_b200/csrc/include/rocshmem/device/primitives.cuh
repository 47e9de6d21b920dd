// Device-side point-to-point primitives over NVLink peer mappings: copies (thread / warp / block),
// put / get / p / g, atomics, signals, bounded waits, ordering.
//
// Reference counterparts: the copy loops memcpy / memcpy_wave / memcpy_wg (src/util.hpp:170-262),
// IPCContext put/get/signal/fence (src/ipc/context_ipc_device.cpp:62-324), the IPC atomics
// (src/ipc_policy.hpp:69-99) and the generic wait_until / test (src/context_tmpl_device.hpp:201-377).
// What differs by design:
//   * a remote address is local + (pe - my_pe) * stride: no table of mapped bases;
//   * copies move 16 bytes per thread per access when source and destination are congruent
//     modulo 16 (the reference moves 8), with several loads in flight per thread;
//   * every atomic family exists for every listed type (the reference's IPC backend leaves swap and
//     the bitwise families unimplemented, src/ipc/context_ipc_tmpl_device.hpp:91-128);
//   * every wait has a budget and reports through the error record instead of spinning for ever;
//   * a host-thread proxy can carry thread-level put/get/atomics when ROCSHMEM_USE_PROXY is set.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../coalesce.h"
#include "state.cuh"

namespace rocshmem {
namespace detail {

// ---- copies ---------------------------------------------------------------------------------------

template <typename V, Scope S>
__device__ __forceinline__ void copy_vec(char *dst, const char *src, size_t nvec, const Group<S> &g) {
  V *d = reinterpret_cast<V *>(dst);
  const V *s = reinterpret_cast<const V *>(src);
  size_t i = g.tid;
  const size_t step = g.size;
  // Four independent loads in flight per thread before the first store.
  for (; i + 3 * step < nvec; i += 4 * step) {
    V a = s[i], b = s[i + step], c = s[i + 2 * step], e = s[i + 3 * step];
    d[i] = a;
    d[i + step] = b;
    d[i + 2 * step] = c;
    d[i + 3 * step] = e;
  }
  for (; i < nvec; i += step) d[i] = s[i];
}

// Copies `bytes` bytes with the threads of group g. Any alignment; the widest vector that both
// addresses allow is used for the body and bytes for the ragged head and tail.
template <Scope S>
__device__ __forceinline__ void copy_bytes(void *dst_v, const void *src_v, size_t bytes,
                                           const Group<S> &g) {
  char *dst = static_cast<char *>(dst_v);
  const char *src = static_cast<const char *>(src_v);
  const uintptr_t d = reinterpret_cast<uintptr_t>(dst), s = reinterpret_cast<uintptr_t>(src);
  const unsigned diff = static_cast<unsigned>((d ^ s) & 15u);
  unsigned width = 16;
  if (diff & 1u) width = 1;
  else if (diff & 2u) width = 2;
  else if (diff & 4u) width = 4;
  else if (diff & 8u) width = 8;
  if (width == 1 || bytes < 32) {
    for (size_t i = g.tid; i < bytes; i += g.size) dst[i] = src[i];
    return;
  }
  size_t head = (width - (d & (width - 1))) & (width - 1);
  if (head > bytes) head = bytes;
  for (size_t i = g.tid; i < head; i += g.size) dst[i] = src[i];
  const size_t nvec = (bytes - head) / width;
  switch (width) {
    case 16: copy_vec<int4, S>(dst + head, src + head, nvec, g); break;
    case 8: copy_vec<int2, S>(dst + head, src + head, nvec, g); break;
    case 4: copy_vec<int, S>(dst + head, src + head, nvec, g); break;
    default: copy_vec<short, S>(dst + head, src + head, nvec, g); break;
  }
  for (size_t i = head + nvec * width + g.tid; i < bytes; i += g.size) dst[i] = src[i];
}

// ---- reverse-offload producer -----------------------------------------------------------------------

// Publishes one command and, when `blocking`, waits for its completion. Returns the fetched value
// (atomics) or 0; *ok tells whether the command completed within the budget.
__device__ inline unsigned long long proxy_submit(unsigned type, int pe, const void *dst,
                                                  const void *src, unsigned long long size,
                                                  unsigned long long cond, unsigned op,
                                                  unsigned dtype_size, bool blocking, bool *ok,
                                                  unsigned long long team_slot = 0) {
  const rocshmem_device_state &s = st();
  rocshmem_proxy_ring *ring = s.proxy;
  *ok = false;
  if (ring == nullptr) return 0;
  SpinBudget budget(s.wait_timeout_ns);
  unsigned long long idx;
  unsigned slot;
  const unsigned long long t_start = prof_now();
  // Reserve an index only once its slot is free (see Proxy::submit for the protocol).
  for (;;) {
    idx = ld_relaxed_sys(ring->write_index);
    slot = static_cast<unsigned>(idx % ring->capacity);
    unsigned long long rd = *ring->read_index;
    if (idx - rd < ring->capacity && ring->cmds[slot].valid == 0) {
      if (atomicCAS(ring->write_index, idx, idx + 1) == idx) break;
      continue;
    }
    if (!budget.keep_going()) {
      record_error(ROCSHMEM_ERR_PROXY_TIMEOUT, pe, 1, ring, idx, rd);
      return 0;
    }
  }
  const unsigned long long t_slot = prof_now();
  stat_add(ROCSHMEM_STAT_PROXY_SLOT_NS, t_slot - t_start);
  rocshmem_proxy_cmd *c = &ring->cmds[slot];
  c->type = type;
  c->pe = pe;
  c->status_slot = blocking ? static_cast<int>(slot) : -1;
  c->dst = reinterpret_cast<unsigned long long>(dst);
  c->src = reinterpret_cast<unsigned long long>(src);
  c->size = size;
  c->cond = cond;
  c->op = op;
  c->dtype_size = dtype_size;
  c->team_slot = team_slot;
  __threadfence_system();
  c->valid = 1;
  __threadfence_system();
  const unsigned long long t_packed = prof_now();
  stat_add(ROCSHMEM_STAT_PROXY_PACK_NS, t_packed - t_slot);
  if (!blocking) {
    *ok = true;
    return 0;
  }
  volatile unsigned long long *status = ring->status + slot;
  unsigned long long fetched = 0;
  bool done = true;
  while (*status < idx + 1) {
    if (!budget.keep_going()) {
      done = false;
      break;
    }
  }
  stat_add(ROCSHMEM_STAT_PROXY_HOST_NS, prof_now() - t_packed);
  if (done) {
    __threadfence_system();
    fetched = ring->fetched[slot];
    c->valid = 0;
  } else {
    record_error(ROCSHMEM_ERR_PROXY_TIMEOUT, pe, 2, c, idx + 1, *status);
    // Not picked up yet: mark cancelled so the consumer retires it; otherwise release the slot.
    if (atomicCAS_system(const_cast<unsigned int *>(&c->valid), 1u, 3u) != 1u) c->valid = 0;
  }
  __threadfence_system();
  *ok = done;
  return fetched;
}

// A thread-level put or get through the proxy. With coalescing on, lanes whose messages form one
// contiguous run to one PE send a single command from the first lane of the run; the others wait for it
// at the warp barrier, so a blocking call still returns only after its bytes have been moved.
__device__ inline void proxy_rma(unsigned type, int pe, void *dest, const void *source, size_t bytes,
                                 bool blocking) {
  bool ok;
  if (!(st().use_proxy & 2)) {
    proxy_submit(type, pe, dest, source, bytes, 0, 0, 1, blocking, &ok);
    return;
  }
  const unsigned active = __activemask();
  coalesce::Msg m{pe, reinterpret_cast<unsigned long long>(dest),
                  reinterpret_cast<unsigned long long>(source), static_cast<unsigned long long>(bytes)};
  if (coalesce::warp_coalesce(m, active)) {
    proxy_submit(type, m.pe, reinterpret_cast<void *>(m.dst), reinterpret_cast<const void *>(m.src), m.size, 0,
                 0, 1, blocking, &ok);
  }
  __syncwarp(active);
}

// ---- put / get ----------------------------------------------------------------------------------------

template <Scope S>
__device__ __forceinline__ void putmem(void *dest, const void *source, size_t bytes, int pe,
                                       bool blocking, bool fence_after) {
  if (bytes == 0) return;
  if (!check_pe(pe, 10) || !check_symmetric(dest, bytes, 10)) return;
  Group<S> g;
  if (g.leader()) stat_add(ROCSHMEM_STAT_BYTES_PUT, bytes);
  if (S == Scope::THREAD && st().use_proxy) {
    proxy_rma(ROCSHMEM_PROXY_PUT, pe, dest, const_cast<void *>(source), bytes, blocking);
    return;
  }
  copy_bytes<S>(remote_ptr(static_cast<char *>(dest), pe), source, bytes, g);
  if (blocking) {
    // Local completion is immediate once the loads of `source` have been consumed; the fence orders
    // this put before later operations of the caller, as the reference's IPC put does.
    if (fence_after) __threadfence_system();
    g.sync();
  }
}

template <Scope S>
__device__ __forceinline__ void getmem(void *dest, const void *source, size_t bytes, int pe,
                                       bool blocking) {
  if (bytes == 0) return;
  if (!check_pe(pe, 11) || !check_symmetric(source, bytes, 11)) return;
  Group<S> g;
  if (g.leader()) stat_add(ROCSHMEM_STAT_BYTES_GET, bytes);
  if (S == Scope::THREAD && st().use_proxy) {
    proxy_rma(ROCSHMEM_PROXY_GET, pe, dest, source, bytes, true);
    return;
  }
  copy_bytes<S>(dest, remote_ptr(static_cast<const char *>(source), pe), bytes, g);
  if (blocking) g.sync();
}

template <typename T>
__device__ __forceinline__ void put_value(T *dest, T value, int pe) {
  if (!check_pe(pe, 12) || !check_symmetric(dest, sizeof(T), 12)) return;
  *reinterpret_cast<volatile T *>(remote_ptr(dest, pe)) = value;
}

template <typename T>
__device__ __forceinline__ T get_value(const T *source, int pe) {
  if (!check_pe(pe, 13) || !check_symmetric(source, sizeof(T), 13)) return T();
  return *reinterpret_cast<const volatile T *>(remote_ptr(source, pe));
}

// ---- atomics --------------------------------------------------------------------------------------------

// Integer types are mapped onto the unsigned type of the same width; the hardware operations are
// identical for signed and unsigned add / exch / cas / and / or / xor.
template <size_t N> struct UIntOf;
template <> struct UIntOf<4> { using type = unsigned int; };
template <> struct UIntOf<8> { using type = unsigned long long; };

template <typename T>
__device__ __forceinline__ typename UIntOf<sizeof(T)>::type to_bits(T v) {
  typename UIntOf<sizeof(T)>::type b;
  memcpy(&b, &v, sizeof(T));
  return b;
}
template <typename T>
__device__ __forceinline__ T from_bits(typename UIntOf<sizeof(T)>::type b) {
  T v;
  memcpy(&v, &b, sizeof(T));
  return v;
}

template <typename T>
__device__ __forceinline__ T amo_fetch_add(T *target, T value, int pe) {
  using U = typename UIntOf<sizeof(T)>::type;
  if (!check_pe(pe, 20) || !check_symmetric(target, sizeof(T), 20)) return T();
  if (st().use_proxy) {
    bool ok;
    return from_bits<T>(static_cast<U>(proxy_submit(ROCSHMEM_PROXY_AMO_FADD, pe, target, nullptr,
                                                    to_bits(value), 0, 0, sizeof(T), true, &ok)));
  }
  return from_bits<T>(atomicAdd_system(reinterpret_cast<U *>(remote_ptr(target, pe)), to_bits(value)));
}
__device__ __forceinline__ float amo_fetch_add(float *target, float value, int pe) {
  if (!check_pe(pe, 20) || !check_symmetric(target, 4, 20)) return 0.f;
  return atomicAdd_system(remote_ptr(target, pe), value);
}
__device__ __forceinline__ double amo_fetch_add(double *target, double value, int pe) {
  if (!check_pe(pe, 20) || !check_symmetric(target, 8, 20)) return 0.0;
  return atomicAdd_system(remote_ptr(target, pe), value);
}

// Any atomic through the reverse-offload ring: `op` is the host's operation code (fetch 0, swap 1, cas 2, add 3,
// and 4, or 5, xor 6). The reference routes every atomic of its reverse-offload backend through the host
// (src/reverse_offload/context_ro_tmpl_device.hpp:210-275).
template <typename T>
__device__ __forceinline__ T amo_via_proxy(unsigned op, T *target, T value, T cond, int pe) {
  using U = typename UIntOf<sizeof(T)>::type;
  bool ok;
  return from_bits<T>(static_cast<U>(proxy_submit(ROCSHMEM_PROXY_AMO, pe, target, nullptr, to_bits(value),
                                                  to_bits(cond), op, sizeof(T), true, &ok)));
}

template <typename T>
__device__ __forceinline__ void amo_add(T *target, T value, int pe) {
  // The result is unused, so the compiler emits the non-returning reduction form.
  (void)amo_fetch_add(target, value, pe);
}

template <typename T>
__device__ __forceinline__ T amo_swap(T *target, T value, int pe) {
  using U = typename UIntOf<sizeof(T)>::type;
  if (!check_pe(pe, 21) || !check_symmetric(target, sizeof(T), 21)) return T();
  if (st().use_proxy) return amo_via_proxy<T>(1, target, value, T(), pe);
  return from_bits<T>(atomicExch_system(reinterpret_cast<U *>(remote_ptr(target, pe)), to_bits(value)));
}

template <typename T>
__device__ __forceinline__ T amo_cas(T *target, T cond, T value, int pe) {
  using U = typename UIntOf<sizeof(T)>::type;
  if (!check_pe(pe, 22) || !check_symmetric(target, sizeof(T), 22)) return T();
  if (st().use_proxy) {
    bool ok;
    return from_bits<T>(static_cast<U>(proxy_submit(ROCSHMEM_PROXY_AMO_CAS, pe, target, nullptr,
                                                    to_bits(value), to_bits(cond), 0, sizeof(T),
                                                    true, &ok)));
  }
  return from_bits<T>(
      atomicCAS_system(reinterpret_cast<U *>(remote_ptr(target, pe)), to_bits(cond), to_bits(value)));
}

template <typename T>
__device__ __forceinline__ T amo_fetch(T *target, int pe) {
  using U = typename UIntOf<sizeof(T)>::type;
  if (!check_pe(pe, 23) || !check_symmetric(target, sizeof(T), 23)) return T();
  if (st().use_proxy) return amo_via_proxy<T>(0, target, T(), T(), pe);
  // An atomic read: OR with zero leaves the value unchanged for every type, including floats.
  return from_bits<T>(atomicOr_system(reinterpret_cast<U *>(remote_ptr(target, pe)), U(0)));
}

template <typename T>
__device__ __forceinline__ T amo_fetch_and(T *target, T value, int pe) {
  using U = typename UIntOf<sizeof(T)>::type;
  if (!check_pe(pe, 24) || !check_symmetric(target, sizeof(T), 24)) return T();
  if (st().use_proxy) return amo_via_proxy<T>(4, target, value, T(), pe);
  return from_bits<T>(atomicAnd_system(reinterpret_cast<U *>(remote_ptr(target, pe)), to_bits(value)));
}
template <typename T>
__device__ __forceinline__ T amo_fetch_or(T *target, T value, int pe) {
  using U = typename UIntOf<sizeof(T)>::type;
  if (!check_pe(pe, 25) || !check_symmetric(target, sizeof(T), 25)) return T();
  if (st().use_proxy) return amo_via_proxy<T>(5, target, value, T(), pe);
  return from_bits<T>(atomicOr_system(reinterpret_cast<U *>(remote_ptr(target, pe)), to_bits(value)));
}
template <typename T>
__device__ __forceinline__ T amo_fetch_xor(T *target, T value, int pe) {
  using U = typename UIntOf<sizeof(T)>::type;
  if (!check_pe(pe, 26) || !check_symmetric(target, sizeof(T), 26)) return T();
  if (st().use_proxy) return amo_via_proxy<T>(6, target, value, T(), pe);
  return from_bits<T>(atomicXor_system(reinterpret_cast<U *>(remote_ptr(target, pe)), to_bits(value)));
}

// ---- ordering ---------------------------------------------------------------------------------------------

// NVLink peer stores are posted writes: a system-scope fence orders them before everything the
// thread does afterwards, and makes them visible to any observer that later acquires a flag written
// by this thread. That is all fence and quiet need; there is no queue to drain.
__device__ __forceinline__ void fence() { __threadfence_system(); }
__device__ __forceinline__ void quiet() { __threadfence_system(); }

// ---- signals ----------------------------------------------------------------------------------------------

__device__ __forceinline__ void signal_op(uint64_t *sig_addr, uint64_t signal, int sig_op, int pe) {
  if (st().use_proxy) {
    // The ring is consumed in order by one host thread, so the signal follows the proxied payload; a payload that
    // this thread (or its group) stored directly is ordered before the command by the fences of the submission.
    bool ok;
    proxy_submit(ROCSHMEM_PROXY_SIGNAL, pe, sig_addr, nullptr, signal, 0, static_cast<unsigned>(sig_op), 8, true, &ok);
    return;
  }
  unsigned long long *r = reinterpret_cast<unsigned long long *>(remote_ptr(sig_addr, pe));
  if (sig_op == ROCSHMEM_SIGNAL_ADD) {
    __threadfence_system();
    atomicAdd_system(r, static_cast<unsigned long long>(signal));
  } else {
    st_release_sys(r, signal);  // release: the payload is visible before the signal
  }
}

template <Scope S>
__device__ __forceinline__ void putmem_signal(void *dest, const void *source, size_t bytes,
                                              uint64_t *sig_addr, uint64_t signal, int sig_op, int pe) {
  if (!check_pe(pe, 30) || !check_symmetric(sig_addr, 8, 30)) return;
  Group<S> g;
  if (bytes != 0 && check_symmetric(dest, bytes, 30)) {
    copy_bytes<S>(remote_ptr(static_cast<char *>(dest), pe), source, bytes, g);
  }
  // Every thread's stores happen-before the leader's release through the group barrier.
  g.sync();
  if (g.leader()) signal_op(sig_addr, signal, sig_op, pe);
  g.sync();
}

template <Scope S>
__device__ __forceinline__ uint64_t signal_fetch(const uint64_t *sig_addr) {
  // Every caller reads the word itself; no broadcast through shared memory is needed.
  return ld_acquire_sys(reinterpret_cast<const unsigned long long *>(sig_addr));
}

// ---- point-to-point synchronisation ------------------------------------------------------------------------

template <typename T>
__device__ __forceinline__ bool compare(T a, int cmp, T b) {
  switch (cmp) {
    case ROCSHMEM_CMP_EQ: return a == b;
    case ROCSHMEM_CMP_NE: return a != b;
    case ROCSHMEM_CMP_GT: return a > b;
    case ROCSHMEM_CMP_GE: return a >= b;
    case ROCSHMEM_CMP_LT: return a < b;
    case ROCSHMEM_CMP_LE: return a <= b;
    default: return false;
  }
}

template <typename T>
__device__ __forceinline__ int test(T *ivar, int cmp, T value) {
  T seen = *reinterpret_cast<volatile T *>(ivar);
  if (compare(seen, cmp, value)) {
    __threadfence_system();  // acquire: later reads see what the signaller wrote before the flag
    return 1;
  }
  return 0;
}

// Returns ROCSHMEM_SUCCESS, or ROCSHMEM_ERROR when the budget ran out (error record written).
template <typename T>
__device__ __forceinline__ int wait_until(T *ivar, int cmp, T value) {
  volatile T *p = reinterpret_cast<volatile T *>(ivar);
  T seen = *p;
  if (!compare(seen, cmp, value)) {
    SpinBudget budget(st().wait_timeout_ns);
    const unsigned long long t_start = prof_now();
    while (!compare(seen = *p, cmp, value)) {
      if (!budget.keep_going()) {
        unsigned long long e = 0, o = 0;
        memcpy(&e, &value, sizeof(T));
        memcpy(&o, &seen, sizeof(T));
        record_error(ROCSHMEM_ERR_WAIT_TIMEOUT, -1, 40, ivar, e, o);
        stat_add(ROCSHMEM_STAT_TIMEOUTS);
        return ROCSHMEM_ERROR;
      }
    }
    stat_add(ROCSHMEM_STAT_WAIT_NS, prof_now() - t_start);
  }
  __threadfence_system();
  return ROCSHMEM_SUCCESS;
}

// `values` points at one operand (VEC == false) or at one operand per element (VEC == true).
template <typename T, bool VEC>
__device__ __forceinline__ void wait_until_all(T *ivars, size_t nelems, const int *status, int cmp,
                                               const T *values) {
  for (size_t i = 0; i < nelems; ++i) {
    if (status && status[i]) continue;
    if (wait_until(ivars + i, cmp, VEC ? values[i] : values[0]) != ROCSHMEM_SUCCESS) return;
  }
}

template <typename T, bool VEC>
__device__ __forceinline__ size_t wait_until_any(T *ivars, size_t nelems, const int *status, int cmp,
                                                 const T *values) {
  if (nelems == 0) return SIZE_MAX;
  bool active = false;
  for (size_t i = 0; i < nelems; ++i) active = active || !(status && status[i]);
  if (!active) return SIZE_MAX;
  SpinBudget budget(st().wait_timeout_ns);
  for (;;) {
    for (size_t i = 0; i < nelems; ++i) {
      if (status && status[i]) continue;
      if (test(ivars + i, cmp, VEC ? values[i] : values[0])) return i;
    }
    if (!budget.keep_going()) {
      record_error(ROCSHMEM_ERR_WAIT_TIMEOUT, -1, 41, ivars, nelems, 0);
      return SIZE_MAX;
    }
  }
}

template <typename T, bool VEC>
__device__ __forceinline__ size_t wait_until_some(T *ivars, size_t nelems, size_t *indices,
                                                  const int *status, int cmp, const T *values) {
  if (nelems == 0) return 0;
  bool active = false;
  for (size_t i = 0; i < nelems; ++i) active = active || !(status && status[i]);
  if (!active) return 0;
  SpinBudget budget(st().wait_timeout_ns);
  for (;;) {
    size_t found = 0;
    for (size_t i = 0; i < nelems; ++i) {
      if (status && status[i]) continue;
      if (test(ivars + i, cmp, VEC ? values[i] : values[0])) indices[found++] = i;
    }
    if (found) return found;
    if (!budget.keep_going()) {
      record_error(ROCSHMEM_ERR_WAIT_TIMEOUT, -1, 42, ivars, nelems, 0);
      return 0;
    }
  }
}

}  // namespace detail
}  // namespace rocshmem
