// Per-module device state and the primitives everything else is built on: symmetric address
// translation, system-scope loads/stores for flags, bounded spinning, error recording.
//
// The reference publishes a Backend* through one __constant__ pointer shared by the whole
// relocatable-device-code library (src/backend_bc.cpp:64-71, src/rocshmem_gpu.cpp:66-68). This
// device API is header-only instead, so each CUDA module (each .cu translation unit) owns a private
// copy of the state in __constant__ memory; a static registration object hands the runtime a
// function that refreshes that copy at rocshmem_init() and whenever the state changes.
#pragma once

#include <cuda_runtime.h>

#include "../rocshmem_common.h"

namespace rocshmem {

// Exported by the runtime library.
void rocshmemx_register_module(void (*upload)(const rocshmem_device_state *, int));

namespace detail {

static __constant__ rocshmem_device_state g_state[ROCSHMEM_MAX_LOCAL_PES];
static __constant__ int g_n_local = 1;

static void upload_state(const rocshmem_device_state *states, int n_local) {
  // Each shared object may carry its own copy of the CUDA runtime; make sure this one works on the
  // device that hosts the PEs before touching the module's symbols.
  // The caller's current device is put back afterwards.
  int previous = -1;
  if (cudaGetDevice(&previous) != cudaSuccess) previous = -1;
  cudaSetDevice(states[0].device_ordinal);
  cudaMemcpyToSymbol(g_state, states, sizeof(rocshmem_device_state) * n_local);
  cudaMemcpyToSymbol(g_n_local, &n_local, sizeof(int));
  if (previous >= 0 && previous != states[0].device_ordinal) cudaSetDevice(previous);
}

struct ModuleRegistration {
  ModuleRegistration() { rocshmemx_register_module(&upload_state); }
};
static ModuleRegistration g_module_registration;

// With several PEs per process a kernel is launched once with gridDim.z == n_local and blockIdx.z
// selects the PE a block belongs to.
__device__ __forceinline__ const rocshmem_device_state &st() {
  return g_state[g_n_local > 1 ? blockIdx.z : 0];
}

// ---- time and spinning ---------------------------------------------------------------------------

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Spin helper: call poll() once per iteration; returns false once the budget is used up. The
// timer is read every 64 polls, and the thread backs off with nanosleep so a long wait does not
// saturate the memory system.
struct SpinBudget {
  unsigned long long deadline;
  unsigned spins;
  __device__ __forceinline__ explicit SpinBudget(unsigned long long budget_ns)
      : deadline(0), spins(0) {
    deadline = now_ns() + budget_ns;
  }
  __device__ __forceinline__ bool keep_going() {
    ++spins;
    if ((spins & 63u) == 0) {
      if (now_ns() > deadline) return false;
      __nanosleep(spins > 4096 ? 256 : 32);
    }
    return true;
  }
};

__device__ __forceinline__ void record_error(uint32_t kind, int pe, int where, const void *addr,
                                             unsigned long long expected,
                                             unsigned long long observed) {
  rocshmem_error_record *e = st().error;
  if (atomicAdd(&e->count, 1u) == 0) {
    e->kind = kind;
    e->pe = pe;
    e->where = where;
    e->addr = reinterpret_cast<unsigned long long>(addr);
    e->expected = expected;
    e->observed = observed;
    __threadfence_system();
  }
}

__device__ __forceinline__ void stat_add(int id, unsigned long long n = 1) {
#ifdef ROCSHMEM_PROFILE
  atomicAdd(&st().stats[id], n);
#else
  (void)id;
  (void)n;
#endif
}

// Time stamp for the *_NS counters: the global timer in profiling builds, 0 (and no timer read) otherwise.
__device__ __forceinline__ unsigned long long prof_now() {
#ifdef ROCSHMEM_PROFILE
  return now_ns();
#else
  return 0;
#endif
}

// ---- system-scope flag accesses -----------------------------------------------------------------

__device__ __forceinline__ void st_release_sys(unsigned long long *p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(unsigned long long *p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u32(unsigned int *p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int *p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// Wait until *p >= target. Returns false on time-out (an error record has been written).
__device__ __forceinline__ bool wait_ge_sys(const unsigned long long *p, unsigned long long target,
                                            int peer, int where, uint32_t kind) {
  unsigned long long seen = ld_acquire_sys(p);
  if (seen >= target) return true;
  SpinBudget budget(st().wait_timeout_ns);
  while ((seen = ld_acquire_sys(p)) < target) {
    if (!budget.keep_going()) {
      record_error(kind, peer, where, p, target, seen);
      return false;
    }
  }
  return true;
}

// ---- addressing -------------------------------------------------------------------------------------

// Address on PE `pe` (world numbering) of the symmetric object at local address `p`.
template <typename T>
__device__ __forceinline__ T *remote_ptr(const T *p, int pe) {
  const rocshmem_device_state &s = st();
  long long delta = (static_cast<long long>(pe) - s.my_pe) * static_cast<long long>(s.heap_stride);
  return reinterpret_cast<T *>(reinterpret_cast<char *>(const_cast<T *>(p)) + delta);
}

// Kernel arguments are identical for all blocks of a launch. When a process hosts several PEs, a
// symmetric address passed to the kernel is the one of the process's first PE; this turns it into
// the address on the block's own PE. With one PE per process it is the identity.
template <typename T>
__device__ __forceinline__ T *local_ptr(T *p) {
  const rocshmem_device_state &s = st();
  return reinterpret_cast<T *>(reinterpret_cast<uintptr_t>(p) + size_t(s.local_index) * s.heap_stride);
}

__device__ __forceinline__ bool check_pe(int pe, int where) {
  const rocshmem_device_state &s = st();
  if (!s.debug_checks) return true;
  if (pe >= 0 && pe < s.n_pes) return true;
  record_error(ROCSHMEM_ERR_BAD_PE, pe, where, nullptr, s.n_pes, pe);
  return false;
}

__device__ __forceinline__ bool check_symmetric(const void *p, size_t bytes, int where) {
  const rocshmem_device_state &s = st();
  if (!s.debug_checks) return true;
  const char *c = static_cast<const char *>(p);
  if (c >= s.heap_base && c + bytes <= s.heap_base + s.heap_stride) return true;
  record_error(ROCSHMEM_ERR_BAD_ADDRESS, -1, where, p, bytes, 0);
  return false;
}

// ---- thread identity inside a block / warp -------------------------------------------------------------

__device__ __forceinline__ unsigned block_tid() {
  return threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
}
__device__ __forceinline__ unsigned block_threads() { return blockDim.x * blockDim.y * blockDim.z; }
__device__ __forceinline__ unsigned lane_id() {
  unsigned l;
  asm("mov.u32 %0, %laneid;" : "=r"(l));
  return l;
}

enum class Scope { THREAD, WARP, BLOCK };

// The set of threads that execute one call together. A warp-level call may be made by a partial
// warp (for example a 16-thread block): the group is the set of lanes that are active at the call.
template <Scope S>
struct Group {
  unsigned tid;
  unsigned size;
  unsigned mask;
  __device__ __forceinline__ Group() {
    if (S == Scope::THREAD) {
      tid = 0;
      size = 1;
      mask = 0;
    } else if (S == Scope::WARP) {
      mask = __activemask();
      size = __popc(mask);
      tid = __popc(mask & ((1u << lane_id()) - 1u));
    } else {
      tid = block_tid();
      size = block_threads();
      mask = 0;
    }
  }
  __device__ __forceinline__ void sync() const {
    if (S == Scope::WARP) __syncwarp(mask);
    if (S == Scope::BLOCK) __syncthreads();
  }
  __device__ __forceinline__ bool leader() const { return tid == 0; }
};

}  // namespace detail
}  // namespace rocshmem

// Debug print from device code, prefixed with the PE and the block; compiled in with -DROCSHMEM_DEBUG_PRINT and
// a no-op otherwise. Device printf emits each call atomically, so no print lock is needed (the reference
// serialises GPU_DPRINTF with a device-wide lock, src/util.hpp:51-71,145-168).
#ifdef ROCSHMEM_DEBUG_PRINT
#include <cstdio>
#define ROCSHMEM_GPU_DPRINTF(fmt, ...) \
  printf("[rocshmem pe %d block %u] " fmt, ::rocshmem::detail::st().my_pe, blockIdx.x, ##__VA_ARGS__)
#else
#define ROCSHMEM_GPU_DPRINTF(fmt, ...) \
  do {                                 \
  } while (0)
#endif
