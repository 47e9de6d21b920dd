// Multi-block collectives on the symmetric heap: barrier, allreduce (one-shot, two-shot, NVLS),
// broadcast, fcollect (all-gather), alltoall. These are the standalone kernels behind the host API
// collectives and the PyTorch ops; the block-collective device API inside user kernels lives in
// rocshmem/device/collectives.cuh.
//
// The reference has no kernels of its own (its collectives are __device__ functions run by one
// work-group inside a user kernel: src/ipc/context_ipc_tmpl_device.hpp:166-531) and performs host
// collectives with MPI (src/host/host_templates.hpp:88-392). Here each collective is one kernel
// over up to 128 blocks per PE:
//   * block b of every PE pairs up through block_pair_barrier, so no block ever waits for another
//     block of its own GPU and the kernels need no grid-wide synchronisation;
//   * data moves as 16-byte NVLink peer loads / stores, with one load per team member in flight per
//     thread (allreduce) or four independent vectors per thread (copies);
//   * allreduce: LL = payloads up to 2 KiB travel as 8-byte words of data + call number, no barrier at all;
//     ONE_SHOT = every PE pulls every source and reduces locally (3 hops, small payloads);
//     TWO_SHOT = PE i reduces slice i from all sources and pushes the result to every dest, which
//     moves (n-1)/n of the payload per direction per GPU, the minimum over point-to-point links;
//     NVLS = multimem.ld_reduce on slice i (the NVSwitch adds the n copies) followed by multimem.st
//     (the switch replicates the result), roughly halving the bytes each GPU puts on its links.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "coll_select.hpp"
#include "kernels.hpp"
#include "launch.cuh"
#include "lib_common.cuh"

namespace rocshmem {
namespace kernels {

namespace {

constexpr unsigned kThreads = 512;
constexpr unsigned kMaxCollBlocks = 128;  // all blocks of a collective are resident at once on 148 SMs
constexpr int OP_RUNTIME = -1;

using detail::Acc;
using detail::from_acc;
using detail::remote_ptr;
using detail::team_pe_to_world;
using detail::to_acc;

template <typename A>
__device__ __forceinline__ A apply_runtime(A a, A b, int op) {
  switch (op) {
    case ROCSHMEM_SUM: return a + b;
    case ROCSHMEM_PROD: return a * b;
    case ROCSHMEM_MIN: return a < b ? a : b;
    case ROCSHMEM_MAX: return a > b ? a : b;
    default: break;
  }
  if constexpr (std::is_integral<A>::value) {
    if (op == ROCSHMEM_AND) return a & b;
    if (op == ROCSHMEM_OR) return a | b;
    if (op == ROCSHMEM_XOR) return a ^ b;
  }
  return b;
}

template <typename T, int OP>
__device__ __forceinline__ typename Acc<T>::type combine(typename Acc<T>::type a,
                                                         typename Acc<T>::type b, int op) {
  if constexpr (OP == ROCSHMEM_SUM) {
    return a + b;
  } else {
    return apply_runtime<typename Acc<T>::type>(a, b, op);
  }
}

// Reduce elements [lo, hi) over all members; the result goes to the local dest only (ALL == false)
// or to every member's dest (ALL == true). `tid`/`nthr` enumerate the threads working on the range.
template <typename T, int OP, bool ALL>
__device__ __forceinline__ void reduce_range(const rocshmem_team_dev *t, T *dest, const T *source,
                                             size_t lo, size_t hi, size_t tid, size_t nthr, int op,
                                             bool aligned) {
  using A = typename Acc<T>::type;
  constexpr int VEC = 16 / sizeof(T);
  const int n = t->size;
  size_t scalar_from = lo;
  if (aligned && (lo % VEC) == 0) {
    const size_t nvec = (hi - lo) / VEC;
    // Two vectors per thread and pass; the loads of both (one per member, up to 8 members at a
    // time) are issued before any value is used.
    constexpr int U = 2;
    for (size_t v = tid; v < nvec; v += U * nthr) {
      size_t e[U];
      bool live[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        live[u] = v + u * nthr < nvec;
        e[u] = lo + (v + u * nthr) * VEC;
      }
      int4 raw[U][8];
      A acc[U][VEC];
      int done = 0;
      bool first = true;
      while (done < n) {
        const int batch = (n - done) < 8 ? (n - done) : 8;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (k < batch) {
            // Start with my own copy, then the peers in rotated order so that at any moment the
            // members read from different sources.
            const int j = (t->my_pe + done + k) % n;
            const int w = team_pe_to_world(t, j);
#pragma unroll
            for (int u = 0; u < U; ++u) {
              if (live[u]) raw[u][k] = ld_global_16(remote_ptr(source + e[u], w));
            }
          }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (k < batch) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
              if (live[u]) {
                const T *x = reinterpret_cast<const T *>(&raw[u][k]);
                if (first && k == 0) {
#pragma unroll
                  for (int q = 0; q < VEC; ++q) acc[u][q] = to_acc<T>(x[q]);
                } else {
#pragma unroll
                  for (int q = 0; q < VEC; ++q) acc[u][q] = combine<T, OP>(acc[u][q], to_acc<T>(x[q]), op);
                }
              }
            }
          }
        }
        first = false;
        done += batch;
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (!live[u]) continue;
        int4 out;
        T *o = reinterpret_cast<T *>(&out);
#pragma unroll
        for (int q = 0; q < VEC; ++q) o[q] = from_acc<T>(acc[u][q]);
        if (ALL) {
          for (int d = 0; d < n; ++d) {
            const int j = (t->my_pe + d) % n;
            st_global_16(remote_ptr(dest + e[u], team_pe_to_world(t, j)), out);
          }
        } else {
          st_global_16(dest + e[u], out);
        }
      }
    }
    scalar_from = lo + nvec * VEC;
  }
  for (size_t e = scalar_from + tid; e < hi; e += nthr) {
    A acc = to_acc<T>(*remote_ptr(source + e, team_pe_to_world(t, 0)));
    for (int j = 1; j < n; ++j) {
      acc = combine<T, OP>(acc, to_acc<T>(*remote_ptr(source + e, team_pe_to_world(t, j))), op);
    }
    T out = from_acc<T>(acc);
    if (ALL) {
      for (int j = 0; j < n; ++j) *remote_ptr(dest + e, team_pe_to_world(t, j)) = out;
    } else {
      dest[e] = out;
    }
  }
}

__global__ void __launch_bounds__(64) barrier_kernel(rocshmem_team_t team) {
  const rocshmem_team_dev *t = detail::team_of(team);
  if (t->my_pe < 0) return;
  // Reuses the device API's block barrier so host- and device-initiated barriers share one epoch. Never through
  // the proxy: this kernel is what the proxy launches for a proxied barrier.
  detail::team_barrier(const_cast<rocshmem_team_dev *>(t), false);
}

template <typename T, int OP>
__global__ void __launch_bounds__(kThreads)
allreduce_one_shot_kernel(rocshmem_team_t team, T *dest_arg, const T *source_arg, size_t nelems, int op) {
  const rocshmem_team_dev *t = detail::team_of(team);
  if (t->my_pe < 0) return;
  T *dest = detail::local_ptr(dest_arg);
  const T *source = detail::local_ptr(const_cast<T *>(source_arg));
  const bool aligned = ((reinterpret_cast<uintptr_t>(dest) | reinterpret_cast<uintptr_t>(source)) & 15u) == 0;
  if (!block_pair_barrier(t, blockIdx.x)) return;
  reduce_range<T, OP, false>(t, dest, source, 0, nelems, size_t(blockIdx.x) * blockDim.x + threadIdx.x,
                             size_t(gridDim.x) * blockDim.x, op, aligned);
  // Nobody overwrites a source while a peer may still be reading it. The result is local, nothing is
  // handed over, so the relaxed form of the barrier is enough.
  block_pair_barrier(t, blockIdx.x, false);
}

template <typename T, int OP>
__global__ void __launch_bounds__(kThreads)
allreduce_two_shot_kernel(rocshmem_team_t team, T *dest_arg, const T *source_arg, size_t nelems, int op) {
  const rocshmem_team_dev *t = detail::team_of(team);
  if (t->my_pe < 0) return;
  T *dest = detail::local_ptr(dest_arg);
  const T *source = detail::local_ptr(const_cast<T *>(source_arg));
  constexpr size_t VEC = 16 / sizeof(T);
  const bool aligned = ((reinterpret_cast<uintptr_t>(dest) | reinterpret_cast<uintptr_t>(source)) & 15u) == 0;
  const size_t n = static_cast<size_t>(t->size);
  size_t per = ((nelems + n - 1) / n + VEC - 1) / VEC * VEC;
  size_t lo = per * static_cast<size_t>(t->my_pe), hi = lo + per;
  if (lo > nelems) lo = nelems;
  if (hi > nelems) hi = nelems;
  if (!block_pair_barrier(t, blockIdx.x)) return;
  reduce_range<T, OP, true>(t, dest, source, lo, hi, size_t(blockIdx.x) * blockDim.x + threadIdx.x,
                            size_t(gridDim.x) * blockDim.x, op, aligned);
  block_pair_barrier(t, blockIdx.x);
}

// ---- NVLS ---------------------------------------------------------------------------------------------

template <typename T>
__device__ __forceinline__ int4 multimem_ld_reduce_add(const void *mc);
template <>
__device__ __forceinline__ int4 multimem_ld_reduce_add<float>(const void *mc) {
  int4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
  return r;
}
template <>
__device__ __forceinline__ int4 multimem_ld_reduce_add<__nv_bfloat16>(const void *mc) {
  int4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
  return r;
}
template <>
__device__ __forceinline__ int4 multimem_ld_reduce_add<__half>(const void *mc) {
  int4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
  return r;
}
__device__ __forceinline__ void multimem_st(void *mc, int4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Teams with a multicast mapping (the world team, and split teams of one PE per process that got an object of
// their own): the switch adds the members' copies. Requires 16-byte aligned buffers and a multiple of 16 bytes
// per slice; the launcher falls back to TWO_SHOT otherwise.
template <typename T>
__global__ void __launch_bounds__(kThreads)
allreduce_nvls_kernel(rocshmem_team_t team, T *dest_arg, const T *source_arg, size_t nelems) {
  const rocshmem_device_state &s = st();
  const rocshmem_team_dev *t = detail::team_of(team);
  if (t->my_pe < 0 || t->mc_base == nullptr) return;
  constexpr size_t VEC = 16 / sizeof(T);
  const size_t n = static_cast<size_t>(t->size);
  const size_t nvec_total = nelems / VEC;  // the launcher guarantees nelems % VEC == 0
  size_t per = (nvec_total + n - 1) / n;
  size_t lo = per * static_cast<size_t>(t->my_pe), hi = lo + per;
  if (lo > nvec_total) lo = nvec_total;
  if (hi > nvec_total) hi = nvec_total;
  const char *src_mc = t->mc_base + (reinterpret_cast<const char *>(detail::local_ptr(const_cast<T *>(source_arg))) - s.heap_base);
  char *dst_mc = t->mc_base + (reinterpret_cast<char *>(detail::local_ptr(dest_arg)) - s.heap_base);
  if (!block_pair_barrier(t, blockIdx.x)) return;
  const size_t tid = size_t(blockIdx.x) * blockDim.x + threadIdx.x, nthr = size_t(gridDim.x) * blockDim.x;
  size_t v = lo + tid;
  for (; v + 3 * nthr < hi; v += 4 * nthr) {
    int4 a = multimem_ld_reduce_add<T>(src_mc + v * 16);
    int4 b = multimem_ld_reduce_add<T>(src_mc + (v + nthr) * 16);
    int4 c = multimem_ld_reduce_add<T>(src_mc + (v + 2 * nthr) * 16);
    int4 d = multimem_ld_reduce_add<T>(src_mc + (v + 3 * nthr) * 16);
    multimem_st(dst_mc + v * 16, a);
    multimem_st(dst_mc + (v + nthr) * 16, b);
    multimem_st(dst_mc + (v + 2 * nthr) * 16, c);
    multimem_st(dst_mc + (v + 3 * nthr) * 16, d);
  }
  for (; v < hi; v += nthr) multimem_st(dst_mc + v * 16, multimem_ld_reduce_add<T>(src_mc + v * 16));
  block_pair_barrier(t, blockIdx.x);
}

// ---- small allreduce without any barrier ---------------------------------------------------------------------------
// Every member stores its payload into its mailbox on every member (itself included) as 8-byte words that carry
// 4 bytes of data and the number of this call: data and "ready" flag arrive in one store, so the receiver needs no
// fence and no flag round trip, and nobody has to wait for anybody before sending. The result is reduced locally in
// member order, hence bit-identical on all members. Two mailboxes per team alternate between calls: a member can be
// at most one call ahead of another (it needs everybody's words of call k to finish call k), so the words of call
// k + 2 never overwrite words of call k that are still being read. One NVLink crossing in total, against the three
// of the one-shot kernel with its two pair barriers. Payloads up to ROCSHMEM_LL_WORDS * 4 bytes, a multiple of 4;
// element types of 2 or 4 bytes.
template <typename T, int OP>
__global__ void __launch_bounds__(kThreads)
allreduce_ll_kernel(rocshmem_team_t team, T *dest_arg, const T *source_arg, size_t nelems, int op) {
  using A = typename Acc<T>::type;
  constexpr int PER = 4 / sizeof(T);  // elements per word
  static_assert(sizeof(T) == 2 || sizeof(T) == 4, "mailbox words carry 4 bytes of data");
  __shared__ unsigned s_epoch;
  const rocshmem_device_state &s = st();
  rocshmem_team_dev *t = const_cast<rocshmem_team_dev *>(detail::team_of(team));
  if (t->my_pe < 0) return;
  unsigned *dest = reinterpret_cast<unsigned *>(detail::local_ptr(dest_arg));
  const unsigned *source = reinterpret_cast<const unsigned *>(detail::local_ptr(const_cast<T *>(source_arg)));
  const int n = t->size, me = t->my_pe;
  const unsigned words = static_cast<unsigned>(nelems / PER);
  if (threadIdx.x == 0) {
    unsigned long long e = t->ll_epoch + 1;
    if ((e & 0xffffffffull) == 0) ++e;   // the flag value 0 means "empty"
    t->ll_epoch = e;
    s_epoch = static_cast<unsigned>(e);
  }
  __syncthreads();
  const unsigned epoch = s_epoch;
  const size_t slot_words = size_t(2) * s.n_pes * ROCSHMEM_LL_WORDS;
  unsigned long long *box = s.ll_buf + size_t(t->slot) * slot_words + size_t(epoch & 1u) * s.n_pes * ROCSHMEM_LL_WORDS;
  for (unsigned w = threadIdx.x; w < words; w += blockDim.x) {
    const unsigned long long word = (static_cast<unsigned long long>(epoch) << 32) | source[w];
    for (int d = 0; d < n; ++d) {
      const int j = (me + d) % n;
      detail::st_relaxed_sys(remote_ptr(box + size_t(me) * ROCSHMEM_LL_WORDS + w, team_pe_to_world(t, j)), word);
    }
  }
  for (unsigned w = threadIdx.x; w < words; w += blockDim.x) {
    A acc[PER];
    bool ok = true;
    for (int j = 0; j < n && ok; ++j) {
      const unsigned long long *p = box + size_t(j) * ROCSHMEM_LL_WORDS + w;
      unsigned long long v = detail::ld_relaxed_sys(p);
      if (static_cast<unsigned>(v >> 32) != epoch) {
        detail::SpinBudget budget(s.wait_timeout_ns);
        while (static_cast<unsigned>((v = detail::ld_relaxed_sys(p)) >> 32) != epoch) {
          if (!budget.keep_going()) {
            detail::record_error(ROCSHMEM_ERR_BARRIER_TIMEOUT, team_pe_to_world(t, j), 63, p, epoch, v);
            ok = false;
            break;
          }
        }
      }
      const unsigned data = static_cast<unsigned>(v);
      const T *x = reinterpret_cast<const T *>(&data);
#pragma unroll
      for (int q = 0; q < PER; ++q) acc[q] = j == 0 ? to_acc<T>(x[q]) : combine<T, OP>(acc[q], to_acc<T>(x[q]), op);
    }
    if (!ok) break;
    unsigned out;
    T *o = reinterpret_cast<T *>(&out);
#pragma unroll
    for (int q = 0; q < PER; ++q) o[q] = from_acc<T>(acc[q]);
    dest[w] = out;
  }
}

// All-gather through the team's NVLink multicast mapping (one PE per process): every 16-byte vector of my
// block is stored once to the multicast address of dest[my_pe * bytes] and the switch delivers it to every member,
// myself included. A member puts `bytes` on its links instead of (n - 1) x bytes.
__global__ void __launch_bounds__(kThreads)
fcollect_nvls_kernel(rocshmem_team_t team, char *dest_arg, const char *source_arg, size_t bytes, int pre_sync) {
  const rocshmem_device_state &s = st();
  const rocshmem_team_dev *t = detail::team_of(team);
  if (t->my_pe < 0 || t->mc_base == nullptr) return;
  char *dest = detail::local_ptr(dest_arg);
  const int4 *src = reinterpret_cast<const int4 *>(detail::local_ptr(const_cast<char *>(source_arg)));
  if (pre_sync && !block_pair_barrier(t, blockIdx.x)) return;
  char *dst_mc = t->mc_base + (dest - s.heap_base) + size_t(t->my_pe) * bytes;
  const size_t nvec = bytes / 16, per = (nvec + gridDim.x - 1) / gridDim.x;
  size_t lo = per * blockIdx.x, hi = lo + per;
  if (lo > nvec) lo = nvec;
  if (hi > nvec) hi = nvec;
  size_t v = lo + threadIdx.x;
  for (; v + 3 * blockDim.x < hi; v += 4 * blockDim.x) {
    const int4 a = src[v], b = src[v + blockDim.x], c = src[v + 2 * blockDim.x], d = src[v + 3 * blockDim.x];
    multimem_st(dst_mc + v * 16, a);
    multimem_st(dst_mc + (v + blockDim.x) * 16, b);
    multimem_st(dst_mc + (v + 2 * blockDim.x) * 16, c);
    multimem_st(dst_mc + (v + 3 * blockDim.x) * 16, d);
  }
  for (; v < hi; v += blockDim.x) multimem_st(dst_mc + v * 16, src[v]);
  block_pair_barrier(t, blockIdx.x);
}

// ---- copies -----------------------------------------------------------------------------------------------

// mode 0: broadcast (root pushes source to every other member's dest)
// mode 1: fcollect  (my source -> dest[my_pe * bytes] on every member)
// mode 2: alltoall  (source[j * bytes] -> dest[my_pe * bytes] on member j)
__global__ void __launch_bounds__(kThreads)
push_kernel(rocshmem_team_t team, char *dest_arg, const char *source_arg, size_t bytes, int root, int mode) {
  const rocshmem_team_dev *t = detail::team_of(team);
  if (t->my_pe < 0) return;
  char *dest = detail::local_ptr(dest_arg);
  const char *source = detail::local_ptr(const_cast<char *>(source_arg));
  const int n = t->size;
  // Optional entry barrier: destinations on every member are known to be free (their previous
  // consumers have finished) before anybody writes into them.
  if (mode & 0x100) {
    if (!block_pair_barrier(t, blockIdx.x)) return;
    mode &= 0xff;
  }
  const bool sender = mode != 0 || t->my_pe == root;
  if (sender) {
    // Each block owns a contiguous share of the payload (multiple of 16 bytes) and sends it to every
    // destination, rotating the order so that the members hit different targets at the same time.
    const size_t share = ((bytes + gridDim.x - 1) / gridDim.x + 15) / 16 * 16;
    size_t lo = share * blockIdx.x, hi = lo + share;
    if (lo > bytes) lo = bytes;
    if (hi > bytes) hi = bytes;
    detail::Group<detail::Scope::BLOCK> g;
    for (int d = 0; d < n && hi > lo; ++d) {
      const int j = (t->my_pe + d) % n;
      if (mode == 0 && j == root) continue;  // the root's own dest stays untouched
      const char *src = source + (mode == 2 ? size_t(j) * bytes : 0) + lo;
      char *dst = dest + (mode == 0 ? 0 : size_t(t->my_pe) * bytes) + lo;
      detail::copy_bytes<detail::Scope::BLOCK>(remote_ptr(dst, team_pe_to_world(t, j)), src, hi - lo, g);
    }
  }
  block_pair_barrier(t, blockIdx.x);
}

// Large broadcast through relays. A root that pushes the whole payload to every member is limited by
// its own NVLink egress ((n - 1) x bytes over one port). Here the payload is cut into sub-chunks and
// each sub-chunk into n - 1 parts, one per non-root member: the root sends part r only to relay r
// (egress = bytes in total), and every relay forwards its part to the other non-root members. The loop
// has one cross-PE barrier per sub-chunk, so the root's send of sub-chunk c + 1 overlaps the relays'
// forwarding of sub-chunk c and all ports stay busy. The root's own dest is left untouched, like in
// the direct variant.
__global__ void __launch_bounds__(kThreads)
broadcast_relay_kernel(rocshmem_team_t team, char *dest_arg, const char *source_arg, size_t bytes, int root,
                       size_t sub_bytes, int pre_sync) {
  const rocshmem_team_dev *t = detail::team_of(team);
  if (t->my_pe < 0) return;
  char *dest = detail::local_ptr(dest_arg);
  const char *source = detail::local_ptr(const_cast<char *>(source_arg));
  const int n = t->size, me = t->my_pe;
  if (pre_sync && !block_pair_barrier(t, blockIdx.x)) return;
  detail::Group<detail::Scope::BLOCK> g;
  const int relays = n - 1;
  const int my_relay = me < root ? me : me - 1;  // meaningless on the root
  for (size_t base = 0; base < bytes; base += sub_bytes) {
    const size_t len = bytes - base < sub_bytes ? bytes - base : sub_bytes;
    const size_t part = ((len + relays - 1) / relays + 15) / 16 * 16;
    const size_t share = ((part + gridDim.x - 1) / gridDim.x + 15) / 16 * 16;
    if (me == root) {
      for (int d = 0; d < relays; ++d) {
        const int r = (d + blockIdx.x) % relays;  // blocks start on different relays
        const int j = r < root ? r : r + 1;
        size_t lo = size_t(r) * part + share * blockIdx.x, hi = lo + share;
        const size_t end = size_t(r + 1) * part < len ? size_t(r + 1) * part : len;
        if (hi > end) hi = end;
        if (lo < hi) {
          detail::copy_bytes<detail::Scope::BLOCK>(remote_ptr(dest + base + lo, team_pe_to_world(t, j)),
                                                   source + base + lo, hi - lo, g);
        }
      }
    }
    // Part r of this sub-chunk has landed on relay r (block b's share of it, on every relay).
    if (!block_pair_barrier(t, blockIdx.x)) return;
    if (me != root) {
      size_t lo = size_t(my_relay) * part + share * blockIdx.x, hi = lo + share;
      const size_t end = size_t(my_relay + 1) * part < len ? size_t(my_relay + 1) * part : len;
      if (hi > end) hi = end;
      for (int d = 1; d < n && lo < hi; ++d) {
        const int j = (me + d) % n;
        if (j == root) continue;
        detail::copy_bytes<detail::Scope::BLOCK>(remote_ptr(dest + base + lo, team_pe_to_world(t, j)),
                                                 dest + base + lo, hi - lo, g);
      }
    }
  }
  block_pair_barrier(t, blockIdx.x);
}

// Large broadcast through the NVLink multicast mapping (world team, one PE per process). The root stores every
// 16-byte vector once to the multicast address of the staging area and the switch delivers it to every member: one
// hop, the root sends the payload once, nobody forwards. The multicast object spans all members, the root included,
// whose own dest must stay as it is, so the payload does not go to dest directly: it lands in the staging area and
// every other member copies it from its local staging into dest (a local copy at HBM speed). Sub-chunks alternate
// between the two halves of the staging area with one cross-PE barrier each, so the members' copy of sub-chunk c
// overlaps the root's stores of sub-chunk c + 1. Block b of every member handles share b of every sub-chunk, which
// is why the pairwise barrier between equal block indices suffices.
__global__ void __launch_bounds__(kThreads)
broadcast_nvls_kernel(rocshmem_team_t team, char *dest_arg, const char *source_arg, size_t bytes, int root,
                      size_t sub_bytes, int pre_sync) {
  const rocshmem_device_state &s = st();
  const rocshmem_team_dev *t = detail::team_of(team);
  if (t->my_pe < 0 || t->mc_base == nullptr) return;
  char *dest = detail::local_ptr(dest_arg);
  const char *source = detail::local_ptr(const_cast<char *>(source_arg));
  if (pre_sync && !block_pair_barrier(t, blockIdx.x)) return;
  const bool is_root = t->my_pe == root;
  char *stage = s.scratch;
  char *stage_mc = t->mc_base + (s.scratch - s.heap_base);  // the same bytes on every member
  int half = 0;
  for (size_t base = 0; base < bytes; base += sub_bytes, half ^= 1) {
    const size_t len = bytes - base < sub_bytes ? bytes - base : sub_bytes;  // a multiple of 16 (launcher)
    // Shares are cut from the full sub-chunk size, also for a shorter last sub-chunk: block b then only ever touches
    // bytes of a staging half that the blocks b of the other members touch, the blocks it synchronises with.
    const size_t nvec = len / 16, per = (sub_bytes / 16 + gridDim.x - 1) / gridDim.x;
    size_t lo = per * blockIdx.x, hi = lo + per;
    if (lo > nvec) lo = nvec;
    if (hi > nvec) hi = nvec;
    const size_t stage_off = size_t(half) * sub_bytes;
    if (is_root) {
      const int4 *src = reinterpret_cast<const int4 *>(source + base);
      size_t v = lo + threadIdx.x;
      for (; v + 3 * blockDim.x < hi; v += 4 * blockDim.x) {
        const int4 a = src[v], b = src[v + blockDim.x], c = src[v + 2 * blockDim.x], d = src[v + 3 * blockDim.x];
        multimem_st(stage_mc + stage_off + v * 16, a);
        multimem_st(stage_mc + stage_off + (v + blockDim.x) * 16, b);
        multimem_st(stage_mc + stage_off + (v + 2 * blockDim.x) * 16, c);
        multimem_st(stage_mc + stage_off + (v + 3 * blockDim.x) * 16, d);
      }
      for (; v < hi; v += blockDim.x) multimem_st(stage_mc + stage_off + v * 16, src[v]);
    }
    // Share b of this sub-chunk has landed in every member's staging half. The half is reused two sub-chunks
    // later, after the barrier of the next one, which a member reaches only when its copy below is done.
    if (!block_pair_barrier(t, blockIdx.x)) return;
    if (!is_root) {
      // Written by another GPU: read past L1, which may still hold the lines of an earlier sub-chunk.
      const int4 *from = reinterpret_cast<const int4 *>(stage + stage_off);
      int4 *to = reinterpret_cast<int4 *>(dest + base);
      size_t v = lo + threadIdx.x;
      for (; v + 3 * blockDim.x < hi; v += 4 * blockDim.x) {
        const int4 a = __ldcg(from + v), b = __ldcg(from + v + blockDim.x), c = __ldcg(from + v + 2 * blockDim.x),
                   d = __ldcg(from + v + 3 * blockDim.x);
        to[v] = a;
        to[v + blockDim.x] = b;
        to[v + 2 * blockDim.x] = c;
        to[v + 3 * blockDim.x] = d;
      }
      for (; v < hi; v += blockDim.x) to[v] = __ldcg(from + v);
    }
  }
  // The staging area belongs to this call until every member has copied its last sub-chunk.
  block_pair_barrier(t, blockIdx.x, false);
}

// ROCSHMEM_BCAST_NVLS=1 lets large broadcasts use the multicast kernel on teams that have a mapping.
bool use_bcast_nvls() {
  static const bool on = [] {
    const char *e = std::getenv("ROCSHMEM_BCAST_NVLS");
    return e != nullptr && e[0] != '\0' && e[0] != '0';
  }();
  return on;
}

// ROCSHMEM_FCOLLECT_NVLS=1 sends all-gathers through the multicast mapping. Off by default: an all-gather is bound
// by what a rank receives, and through the switch it receives its own block as well (n blocks instead of n - 1),
// so the push kernel is faster wherever both were measured (64 MiB per member: 131 us against 208 us on two GPUs,
// 324 us against 388 us on four); what the switch saves is egress, (n - 1) blocks down to one.
bool use_fcollect_nvls() {
  static const bool on = [] {
    const char *e = std::getenv("ROCSHMEM_FCOLLECT_NVLS");
    return e != nullptr && e[0] != '\0' && e[0] != '0';
  }();
  return on;
}

template <typename K>
unsigned clamp_blocks(K kernel, unsigned want) {
  Runtime &rt = Runtime::instance();
  unsigned b = std::min<unsigned>(want, kMaxCollBlocks);
  if (rt.n_local() > 1) b = std::min(b, coresident_blocks_per_pe(kernel, kThreads, 0, rt.n_local()));
  return std::max(1u, b);
}

template <typename T>
int launch_allreduce_typed(rocshmem_team_t team, void *dest, const void *source, size_t nelems, int op,
                           int algo, cudaStream_t stream) {
  const size_t bytes = nelems * sizeof(T);
  Runtime &rt = Runtime::instance();
  HostTeam *ht = rt.team_from_handle(team);
  const int n = ht ? ht->world.size : rt.n_pes();
  constexpr bool kMultimem = std::is_same<T, float>::value || std::is_same<T, __half>::value ||
                             std::is_same<T, __nv_bfloat16>::value;
  AllreduceRequest req{algo, bytes, sizeof(T), n, ht != nullptr && ht->mc_window != nullptr, op == ROCSHMEM_SUM, kMultimem,
                       reinterpret_cast<uintptr_t>(dest), reinterpret_cast<uintptr_t>(source)};
  algo = select_allreduce(req);
  if (algo == ALLREDUCE_LL) {
    if constexpr (sizeof(T) == 2 || sizeof(T) == 4) {
      const unsigned words = static_cast<unsigned>(bytes / 4);
      const unsigned threads = std::min(kThreads, std::max(32u, (words + 31) / 32 * 32));
      auto k = op == ROCSHMEM_SUM ? allreduce_ll_kernel<T, ROCSHMEM_SUM> : allreduce_ll_kernel<T, OP_RUNTIME>;
      return launch_pes(k, 1, threads, 0, stream, false, team, static_cast<T *>(dest), static_cast<const T *>(source),
                        nelems, op);
    } else {
      return cudaErrorInvalidValue;   // select_allreduce never picks it for other element sizes
    }
  }
  const unsigned want = static_cast<unsigned>(coll_blocks_for(algo == ALLREDUCE_ONE_SHOT ? bytes : bytes / n));
  T *d = static_cast<T *>(dest);
  const T *s = static_cast<const T *>(source);
  if (algo == ALLREDUCE_NVLS) {
    if constexpr (std::is_same<T, float>::value || std::is_same<T, __half>::value ||
                  std::is_same<T, __nv_bfloat16>::value) {
      auto k = allreduce_nvls_kernel<T>;
      return launch_pes(k, clamp_blocks(k, want), kThreads, 0, stream, false, team, d, s, nelems);
    }
  }
  const bool sum = op == ROCSHMEM_SUM;
  if (algo == ALLREDUCE_ONE_SHOT) {
    auto k = sum ? allreduce_one_shot_kernel<T, ROCSHMEM_SUM> : allreduce_one_shot_kernel<T, OP_RUNTIME>;
    return launch_pes(k, clamp_blocks(k, want), kThreads, 0, stream, false, team, d, s, nelems, op);
  }
  auto k = sum ? allreduce_two_shot_kernel<T, ROCSHMEM_SUM> : allreduce_two_shot_kernel<T, OP_RUNTIME>;
  return launch_pes(k, clamp_blocks(k, want), kThreads, 0, stream, false, team, d, s, nelems, op);
}

}  // namespace

int coll_blocks_for(size_t bytes) {
  // One block per 8 KiB of payload (one 16-byte vector per thread of a 512-thread block), between
  // 1 and 128: a remote access costs about 2 us whatever its size, so a block should not have to
  // make several dependent round trips while other SMs sit idle.
  size_t b = (bytes + (size_t(8) << 10) - 1) / (size_t(8) << 10);
  if (b < 1) b = 1;
  if (b > kMaxCollBlocks) b = kMaxCollBlocks;
  return static_cast<int>(b);
}

bool nvls_available() { return Runtime::initialized() && Runtime::instance().mc_base() != nullptr; }

namespace {
template <typename K>
void load_now(K kernel, int *rc) {
  cudaFuncAttributes attr;
  cudaError_t e = cudaFuncGetAttributes(&attr, kernel);
  if (e != cudaSuccess && *rc == 0) *rc = static_cast<int>(e);
}
template <typename T>
void load_allreduce_now(int *rc) {
  if constexpr (sizeof(T) == 2 || sizeof(T) == 4) {
    load_now(allreduce_ll_kernel<T, ROCSHMEM_SUM>, rc);
    load_now(allreduce_ll_kernel<T, OP_RUNTIME>, rc);
  }
  load_now(allreduce_one_shot_kernel<T, ROCSHMEM_SUM>, rc);
  load_now(allreduce_one_shot_kernel<T, OP_RUNTIME>, rc);
  load_now(allreduce_two_shot_kernel<T, ROCSHMEM_SUM>, rc);
  load_now(allreduce_two_shot_kernel<T, OP_RUNTIME>, rc);
}
}  // namespace

// With lazy module loading the first launch of a kernel may have to wait for the kernels that are running. The
// proxy thread launches these collectives precisely while a user kernel waits for their completion, so a process
// that runs device collectives through the proxy loads all of them up front.
int coll_preload() {
  int rc = 0;
  load_now(barrier_kernel, &rc);
  load_now(push_kernel, &rc);
  load_now(broadcast_relay_kernel, &rc);
  load_now(broadcast_nvls_kernel, &rc);
  load_now(fcollect_nvls_kernel, &rc);
  load_allreduce_now<short>(&rc);
  load_allreduce_now<int>(&rc);
  load_allreduce_now<long long>(&rc);
  load_allreduce_now<unsigned int>(&rc);
  load_allreduce_now<unsigned long long>(&rc);
  load_allreduce_now<float>(&rc);
  load_allreduce_now<double>(&rc);
  load_allreduce_now<__half>(&rc);
  load_allreduce_now<__nv_bfloat16>(&rc);
  load_now(allreduce_nvls_kernel<float>, &rc);
  load_now(allreduce_nvls_kernel<__half>, &rc);
  load_now(allreduce_nvls_kernel<__nv_bfloat16>, &rc);
  return rc;
}

int coll_barrier(rocshmem_team_t team, void *stream) {
  return launch_pes(barrier_kernel, 1, 64, 0, static_cast<cudaStream_t>(stream), false, team);
}

int coll_allreduce(rocshmem_team_t team, void *dest, const void *source, size_t nelems, int dtype, int op,
                   int algo, void *stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (nelems == 0) return 0;
  switch (dtype) {
    case ROCSHMEM_I16: return launch_allreduce_typed<short>(team, dest, source, nelems, op, algo, stream);
    case ROCSHMEM_I32: return launch_allreduce_typed<int>(team, dest, source, nelems, op, algo, stream);
    case ROCSHMEM_I64: return launch_allreduce_typed<long long>(team, dest, source, nelems, op, algo, stream);
    case ROCSHMEM_U32: return launch_allreduce_typed<unsigned int>(team, dest, source, nelems, op, algo, stream);
    case ROCSHMEM_U64: return launch_allreduce_typed<unsigned long long>(team, dest, source, nelems, op, algo, stream);
    case ROCSHMEM_F32: return launch_allreduce_typed<float>(team, dest, source, nelems, op, algo, stream);
    case ROCSHMEM_F64: return launch_allreduce_typed<double>(team, dest, source, nelems, op, algo, stream);
    case ROCSHMEM_F16: return launch_allreduce_typed<__half>(team, dest, source, nelems, op, algo, stream);
    case ROCSHMEM_BF16: return launch_allreduce_typed<__nv_bfloat16>(team, dest, source, nelems, op, algo, stream);
    default: return cudaErrorInvalidValue;
  }
}

static int launch_push(rocshmem_team_t team, void *dest, const void *source, size_t bytes, int root,
                       int mode, void *stream, int flags) {
  if (bytes == 0) return 0;
  if (flags & COLL_PRE_SYNC) mode |= 0x100;
  unsigned blocks = clamp_blocks(push_kernel, static_cast<unsigned>(coll_blocks_for(bytes)));
  return launch_pes(push_kernel, blocks, kThreads, 0, static_cast<cudaStream_t>(stream), false, team,
                    static_cast<char *>(dest), static_cast<const char *>(source), bytes, root, mode);
}

int coll_broadcast(rocshmem_team_t team, void *dest, const void *source, size_t bytes, int root,
                   void *stream, int flags) {
  Runtime &rt = Runtime::instance();
  HostTeam *ht = rt.team_from_handle(team);
  const int n = ht ? ht->world.size : 0;
  const bool aligned16 = reinterpret_cast<uintptr_t>(dest) % 16 == 0 && reinterpret_cast<uintptr_t>(source) % 16 == 0;
  const BroadcastPlan plan = plan_broadcast(bytes, n, use_bcast_nvls(), ht != nullptr && ht->mc_window != nullptr,
                                            rt.n_local(), aligned16, rt.config().scratch_size);
  if (plan.kind == BROADCAST_NVLS) {
    // Two staging halves of one sub-chunk each.
    unsigned blocks = clamp_blocks(broadcast_nvls_kernel, static_cast<unsigned>(coll_blocks_for(plan.sub_bytes)));
    return launch_pes(broadcast_nvls_kernel, blocks, kThreads, 0, static_cast<cudaStream_t>(stream), false, team,
                      static_cast<char *>(dest), static_cast<const char *>(source), bytes, root, plan.sub_bytes,
                      (flags & COLL_PRE_SYNC) ? 1 : 0);
  }
  if (plan.kind == BROADCAST_RELAY) {
    unsigned blocks = clamp_blocks(broadcast_relay_kernel,
                                   static_cast<unsigned>(coll_blocks_for(plan.sub_bytes / (n - 1))));
    return launch_pes(broadcast_relay_kernel, blocks, kThreads, 0, static_cast<cudaStream_t>(stream), false, team,
                      static_cast<char *>(dest), static_cast<const char *>(source), bytes, root, plan.sub_bytes,
                      (flags & COLL_PRE_SYNC) ? 1 : 0);
  }
  return launch_push(team, dest, source, bytes, root, 0, stream, flags);
}
int coll_fcollect(rocshmem_team_t team, void *dest, const void *source, size_t bytes, void *stream,
                  int flags) {
  Runtime &rt = Runtime::instance();
  HostTeam *ht = rt.team_from_handle(team);
  if (use_fcollect_nvls() && ht != nullptr && rt.n_local() == 1 && ht->mc_window != nullptr &&
      ht->world.size >= 2 && bytes >= 4096 && bytes % 16 == 0 && reinterpret_cast<uintptr_t>(dest) % 16 == 0 &&
      reinterpret_cast<uintptr_t>(source) % 16 == 0) {
    unsigned blocks = clamp_blocks(fcollect_nvls_kernel, static_cast<unsigned>(coll_blocks_for(bytes)));
    return launch_pes(fcollect_nvls_kernel, blocks, kThreads, 0, static_cast<cudaStream_t>(stream), false, team,
                      static_cast<char *>(dest), static_cast<const char *>(source), bytes,
                      (flags & COLL_PRE_SYNC) ? 1 : 0);
  }
  return launch_push(team, dest, source, bytes, 0, 1, stream, flags);
}
int coll_alltoall(rocshmem_team_t team, void *dest, const void *source, size_t bytes, void *stream,
                  int flags) {
  return launch_push(team, dest, source, bytes, 0, 2, stream, flags);
}

}  // namespace kernels
}  // namespace rocshmem
