// Host-API engine for the CUDA backend: stream-ordered copies on peer-mapped addresses plus small
// helper kernels, so that host-initiated operations use the same NVLink path and the same
// system-scope semantics as device-initiated ones.
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <stdexcept>
#include <string>
#include <thread>

#include "../kernels/kernels.hpp"
#include "../kernels/launch.cuh"
#include "host_ops.hpp"
#include "rocshmem/rocshmem.h"
#include "runtime.hpp"

namespace rocshmem {

namespace {

void check(cudaError_t e, const char *what) {
  if (e != cudaSuccess) {
    throw std::runtime_error(std::string("rocshmem host API: ") + what + ": " + cudaGetErrorString(e));
  }
}

// One atomic on behalf of the host. `target` is already the address on the destination PE.
template <typename U>
__device__ U host_amo_apply(U *target, int op, U value, U cond) {
  switch (op) {
    case ROCSHMEM_AMO_FETCH: return atomicOr_system(target, U(0));
    case ROCSHMEM_AMO_SWAP: return atomicExch_system(target, value);
    case ROCSHMEM_AMO_CAS: return atomicCAS_system(target, cond, value);
    case ROCSHMEM_AMO_ADD: return atomicAdd_system(target, value);
    case ROCSHMEM_AMO_AND: return atomicAnd_system(target, value);
    case ROCSHMEM_AMO_OR: return atomicOr_system(target, value);
    case ROCSHMEM_AMO_XOR: return atomicXor_system(target, value);
    default: return U(0);
  }
}

__global__ void host_amo_kernel(int op, int dtype, void *target, unsigned long long value,
                                unsigned long long cond, unsigned long long *result) {
  unsigned long long old = 0;
  if (dtype == ROCSHMEM_F32 && op == ROCSHMEM_AMO_ADD) {
    float add = __uint_as_float(static_cast<unsigned int>(value));
    old = __float_as_uint(atomicAdd_system(static_cast<float *>(target), add));
  } else if (dtype == ROCSHMEM_F64 && op == ROCSHMEM_AMO_ADD) {
    double add = __longlong_as_double(static_cast<long long>(value));
    old = static_cast<unsigned long long>(
        __double_as_longlong(atomicAdd_system(static_cast<double *>(target), add)));
  } else if (dtype == ROCSHMEM_I32 || dtype == ROCSHMEM_U32 || dtype == ROCSHMEM_F32) {
    old = host_amo_apply<unsigned int>(static_cast<unsigned int *>(target), op,
                                       static_cast<unsigned int>(value), static_cast<unsigned int>(cond));
  } else {
    old = host_amo_apply<unsigned long long>(static_cast<unsigned long long *>(target), op, value, cond);
  }
  __threadfence_system();
  *result = old;
}

// Host threads start with device 0 current. Every entry point of the engine may be the first CUDA call of a user
// thread, so each selects the runtime's device for its own duration and puts the caller's choice back.
class DeviceScope {
 public:
  explicit DeviceScope(int want) {
    int cur = -1;
    if (cudaGetDevice(&cur) == cudaSuccess && cur != want && cudaSetDevice(want) == cudaSuccess) prev_ = cur;
  }
  ~DeviceScope() {
    if (prev_ >= 0) cudaSetDevice(prev_);
  }
  DeviceScope(const DeviceScope &) = delete;
  DeviceScope &operator=(const DeviceScope &) = delete;

 private:
  int prev_ = -1;
};

class CudaHostOps final : public HostOps {
 public:
  explicit CudaHostOps(Runtime *rt) : rt_(rt) {
    check(cudaSetDevice(rt->device()), "cudaSetDevice");
    check(cudaHostAlloc(reinterpret_cast<void **>(&slots_), 4096, cudaHostAllocMapped | cudaHostAllocPortable),
          "pinned result slots");
    check(cudaStreamCreateWithFlags(&poll_stream_, cudaStreamNonBlocking), "poll stream");
    // Load the helper kernel now. With lazy module loading its first launch could otherwise have to wait for
    // running kernels, and the proxy thread launches it precisely while a kernel waits for its result.
    cudaFuncAttributes attr;
    check(cudaFuncGetAttributes(&attr, host_amo_kernel), "helper kernel load");
    if (rt->config().use_proxy && rt->config().proxy_collectives) {
      check(static_cast<cudaError_t>(kernels::coll_preload()), "collective kernel load");
    }
  }
  ~CudaHostOps() override {
    if (slots_) cudaFreeHost(slots_);
    if (poll_stream_) cudaStreamDestroy(poll_stream_);
  }

  void ctx_init(HostCtx *c) override {
    DeviceScope on_device(rt_->device());
    cudaStream_t s;
    check(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "context stream");
    c->stream = s;
  }
  void ctx_fini(HostCtx *c) override {
    DeviceScope on_device(rt_->device());
    if (c->stream) {
      cudaStreamSynchronize(stream(c));
      cudaStreamDestroy(stream(c));
      c->stream = nullptr;
    }
  }

  void put(HostCtx *c, void *dst, const void *src, size_t bytes, int pe, bool blocking) override {
    DeviceScope on_device(rt_->device());
    check(cudaMemcpyAsync(rt_->translate(dst, pe), src, bytes, cudaMemcpyDefault, stream(c)), "put");
    if (blocking) check(cudaStreamSynchronize(stream(c)), "put completion");
  }
  void get(HostCtx *c, void *dst, const void *src, size_t bytes, int pe, bool blocking) override {
    DeviceScope on_device(rt_->device());
    check(cudaMemcpyAsync(dst, rt_->translate(src, pe), bytes, cudaMemcpyDefault, stream(c)), "get");
    if (blocking) check(cudaStreamSynchronize(stream(c)), "get completion");
  }

  uint64_t amo(HostCtx *c, AmoOp op, DType t, void *target, uint64_t value, uint64_t cond, int pe) override {
    DeviceScope on_device(rt_->device());
    // One result word per calling thread: threads with contexts of their own do not wait for one another.
    const unsigned slot = my_slot();
    std::lock_guard<std::mutex> g(slot_mu_[slot]);
    unsigned long long *result = slots_ + slot;
    host_amo_kernel<<<1, 1, 0, stream(c)>>>(static_cast<int>(op), static_cast<int>(t),
                                            rt_->translate(target, pe), value, cond, result);
    check(cudaGetLastError(), "atomic launch");
    check(cudaStreamSynchronize(stream(c)), "atomic completion");
    return *result;
  }

  // Operations of one context are stream-ordered, which is stronger than fence requires.
  void fence(HostCtx *) override {}
  void quiet(HostCtx *c) override {
    DeviceScope on_device(rt_->device());
    check(cudaStreamSynchronize(stream(c)), "quiet");
  }

  int test(void *ivar, DType t, int cmp, uint64_t value) override {
    DeviceScope on_device(rt_->device());
    uint64_t seen = peek(ivar, dtype_size(t));
    return compare_bits(seen, t, cmp, value) ? 1 : 0;
  }

  // Polls with small device-to-host copies instead of parking a kernel on the GPU: the GPU stays
  // free for the work that will eventually satisfy the wait.
  int wait_until(void *ivar, DType t, int cmp, uint64_t value) override {
    DeviceScope on_device(rt_->device());
    auto deadline = std::chrono::steady_clock::now() +
                    std::chrono::milliseconds(rt_->config().wait_timeout_ms);
    uint64_t seen = 0;
    for (;;) {
      seen = peek(ivar, dtype_size(t));
      if (compare_bits(seen, t, cmp, value)) return ROCSHMEM_SUCCESS;
      if (std::chrono::steady_clock::now() > deadline) break;
      std::this_thread::yield();
    }
    rocshmem_error_record e{};
    e.count = 1;
    e.kind = ROCSHMEM_ERR_WAIT_TIMEOUT;
    e.pe = -1;
    e.addr = reinterpret_cast<uint64_t>(ivar);
    e.expected = value;
    e.observed = seen;
    rocshmem_error_record cur = rt_->read_error();
    if (cur.count == 0) {
      rt_->mem().write(rt_->internal_base(rt_->my_pe()) + rt_->layout().error, &e, sizeof(e));
    }
    rt_->count(ROCSHMEM_STAT_TIMEOUTS);
    return ROCSHMEM_ERROR;
  }

  int barrier(HostCtx *c, HostTeam *team, bool sync_only) override {
    DeviceScope on_device(rt_->device());
    // barrier_all completes the context's outstanding operations first; stream order does that.
    (void)sync_only;
    unsigned before = error_count();
    check(static_cast<cudaError_t>(kernels::coll_barrier(team->dev, stream(c))), "barrier launch");
    check(cudaStreamSynchronize(stream(c)), "barrier completion");
    return error_count() == before ? ROCSHMEM_SUCCESS : ROCSHMEM_ERROR;
  }

  int broadcast(HostCtx *c, HostTeam *team, void *dst, const void *src, size_t bytes, int root) override {
    DeviceScope on_device(rt_->device());
    return run(c, kernels::coll_broadcast(team->dev, to_first(dst), to_first(src), bytes, root, stream(c),
                                          kernels::COLL_PRE_SYNC));
  }
  int reduce(HostCtx *c, HostTeam *team, void *dst, const void *src, size_t nelems, DType t,
             ROCSHMEM_OP op) override {
    DeviceScope on_device(rt_->device());
    return run(c, kernels::coll_allreduce(team->dev, to_first(dst), to_first(src), nelems,
                                          static_cast<int>(t), op, kernels::ALLREDUCE_AUTO, stream(c)));
  }
  int fcollect(HostCtx *c, HostTeam *team, void *dst, const void *src, size_t bytes) override {
    DeviceScope on_device(rt_->device());
    return run(c, kernels::coll_fcollect(team->dev, to_first(dst), to_first(src), bytes, stream(c),
                                         kernels::COLL_PRE_SYNC));
  }
  int alltoall(HostCtx *c, HostTeam *team, void *dst, const void *src, size_t bytes) override {
    DeviceScope on_device(rt_->device());
    return run(c, kernels::coll_alltoall(team->dev, to_first(dst), to_first(src), bytes, stream(c),
                                         kernels::COLL_PRE_SYNC));
  }

 private:
  static cudaStream_t stream(HostCtx *c) { return static_cast<cudaStream_t>(c->stream); }

  // Kernels take the address on the process's first local PE and rebase per block.
  void *to_first(const void *p) { return rt_->translate(p, rt_->first_pe()); }

  unsigned error_count() {
    unsigned total = 0;
    for (int l = 0; l < rt_->n_local(); ++l) total += rt_->read_error(l).count;
    return total;
  }

  int run(HostCtx *c, int launch_rc) {
    unsigned before = error_count();
    check(static_cast<cudaError_t>(launch_rc), "collective launch");
    check(cudaStreamSynchronize(stream(c)), "collective completion");
    return error_count() == before ? ROCSHMEM_SUCCESS : ROCSHMEM_ERROR;
  }

  uint64_t peek(const void *p, size_t bytes) {
    const unsigned index = my_slot();
    std::lock_guard<std::mutex> g(slot_mu_[index]);
    unsigned long long *slot = slots_ + kSlots + index;
    *slot = 0;
    check(cudaMemcpyAsync(slot, p, bytes, cudaMemcpyDeviceToHost, poll_stream_), "poll copy");
    check(cudaStreamSynchronize(poll_stream_), "poll completion");
    return *slot;
  }

  // Threads take result words round robin; two threads share one (and its lock) only beyond kSlots threads.
  static constexpr unsigned kSlots = 240;   // 2 x 240 words of 8 bytes fit the 4 KiB allocation
  unsigned my_slot() {
    thread_local unsigned mine = next_slot_.fetch_add(1, std::memory_order_relaxed) % kSlots;
    return mine;
  }

  Runtime *rt_;
  unsigned long long *slots_ = nullptr;
  cudaStream_t poll_stream_ = nullptr;
  std::mutex slot_mu_[kSlots];
  std::atomic<unsigned> next_slot_{0};
};

}  // namespace

HostOps *make_cuda_host_ops(Runtime *rt) { return new CudaHostOps(rt); }

namespace kernels {
int host_amo(int op, int dtype, void *target, uint64_t value, uint64_t cond, uint64_t *result, void *stream) {
  host_amo_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
      op, dtype, target, value, cond, reinterpret_cast<unsigned long long *>(result));
  return cudaGetLastError();
}
}  // namespace kernels

}  // namespace rocshmem
