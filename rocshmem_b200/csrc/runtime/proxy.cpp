#include "proxy.hpp"

#include <cuda_runtime_api.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>

#include "host_ops.hpp"
#include "rocshmem/coalesce.h"
#include "runtime.hpp"

namespace rocshmem {

namespace {
DType dtype_for_size(unsigned int bytes) { return bytes == 4 ? DType::U32 : DType::U64; }
}  // namespace

Proxy::Proxy(Runtime *rt) : rt_(rt) {}

Proxy::~Proxy() { stop(); }

void Proxy::start() {
  if (running_.load()) return;
  const unsigned cap = static_cast<unsigned>(rt_->config().proxy_queue_size);
  size_t cmds_bytes = sizeof(rocshmem_proxy_cmd) * cap;
  size_t words = size_t(cap) * 2 + 16;
  ring_bytes_ = cmds_bytes + words * sizeof(unsigned long long);
  pinned_ = rt_->is_cuda() && rt_->config().proxy_on_cpu;
  if (rt_->is_cuda()) {
    // Pinned and mapped: the same address is valid on the GPU under unified addressing.
    if (cudaHostAlloc(&ring_mem_, ring_bytes_, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
      cudaGetLastError();
      throw std::runtime_error("proxy: cannot allocate the pinned command ring");
    }
    pinned_ = true;
  } else {
    ring_mem_ = std::aligned_alloc(256, (ring_bytes_ + 255) / 256 * 256);
    if (!ring_mem_) throw std::runtime_error("proxy: cannot allocate the command ring");
  }
  std::memset(ring_mem_, 0, ring_bytes_);
  char *base = static_cast<char *>(ring_mem_);
  ring_.cmds = reinterpret_cast<rocshmem_proxy_cmd *>(base);
  ring_.capacity = cap;
  ring_.n_status = cap;
  auto *w = reinterpret_cast<unsigned long long *>(base + cmds_bytes);
  ring_.read_index = w;
  ring_.status = w + 8;
  ring_.fetched = w + 8 + cap;
  // The reservation counter is bumped with device atomics, so it lives in device memory next to the
  // device-visible copy of the ring header. All PEs of this process produce into the one ring, so they
  // share one counter (the first local PE's); a counter per PE would hand the same slots out twice.
  char *counter = rt_->internal_base(rt_->first_pe()) + rt_->layout().proxy + 128;
  rt_->mem().zero(counter, 8);
  for (int l = 0; l < rt_->n_local(); ++l) {
    char *ib = rt_->internal_base(rt_->first_pe() + l) + rt_->layout().proxy;
    rocshmem_proxy_ring dev = ring_;
    dev.write_index = reinterpret_cast<unsigned long long *>(counter);
    rt_->mem().write(ib, &dev, sizeof(dev));
  }
  ring_.write_index = nullptr;
  read_ = 0;
  host_write_.store(0);
  stop_.store(false);
  coalesce_.store(rt_->config().proxy_coalesce != 0);
  running_.store(true);
  thread_ = std::thread([this] { run(); });
}

void Proxy::stop() {
  if (!running_.load()) return;
  stop_.store(true);
  if (thread_.joinable()) thread_.join();
  running_.store(false);
  if (ring_mem_) {
    if (pinned_) {
      cudaFreeHost(ring_mem_);
    } else {
      std::free(ring_mem_);
    }
    ring_mem_ = nullptr;
  }
}

void Proxy::run() {
  // The consumer thread issues CUDA work, so it selects the runtime's device first.
  if (rt_->is_cuda()) cudaSetDevice(rt_->device());
  unsigned idle = 0;
  while (!stop_.load(std::memory_order_relaxed)) {
    rocshmem_proxy_cmd &slot = ring_.cmds[read_ % ring_.capacity];
    unsigned v = __atomic_load_n(&slot.valid, __ATOMIC_ACQUIRE);
    if (v == 3) {
      // Cancelled by a producer whose wait ran out before the command was picked up.
      __atomic_store_n(&slot.valid, 0u, __ATOMIC_RELEASE);
      ++read_;
      __atomic_store_n(const_cast<unsigned long long *>(ring_.read_index),
                       static_cast<unsigned long long>(read_), __ATOMIC_RELEASE);
      continue;
    }
    if (v != 1) {
      if (++idle > 2000) std::this_thread::sleep_for(std::chrono::microseconds(20));
      continue;
    }
    idle = 0;
    // Claim the command with a compare-and-swap: a producer whose wait ran out may be cancelling it (1 -> 3) at
    // this very moment, and a plain store would overwrite the cancellation and leave the slot claimed for ever.
    unsigned expect_published = 1;
    if (!__atomic_compare_exchange_n(&slot.valid, &expect_published, 2u, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE)) {
      continue;   // cancelled in the meantime: the next iteration retires it
    }
    rocshmem_proxy_cmd cmd;
    std::memcpy(&cmd, const_cast<rocshmem_proxy_cmd *>(&slot), sizeof(cmd));
    uint64_t seq = read_ + 1;
    int d = delay_ms_.load();
    if (d > 0) std::this_thread::sleep_for(std::chrono::milliseconds(d));
    int drop = drop_.load();
    bool dropped = false;
    while (drop > 0) {
      if (drop_.compare_exchange_weak(drop, drop - 1)) {
        dropped = true;
        break;
      }
    }
    if (dropped) {
      // Injected loss: the command is retired without being executed or acknowledged. A blocking
      // producer runs into its time-out and frees the slot itself.
      dropped_count_.fetch_add(1);
      if (cmd.status_slot < 0) __atomic_store_n(&slot.valid, 0u, __ATOMIC_RELEASE);
    } else {
      // Commands behind this one that continue it (published already, same kind and PE, equal sizes, both
      // addresses following on) are executed as part of it and then acknowledged one by one.
      unsigned extra = 0;
      if (coalesce_.load(std::memory_order_relaxed) &&
          (cmd.type == ROCSHMEM_PROXY_PUT || cmd.type == ROCSHMEM_PROXY_GET)) {
        coalesce::Msg last{cmd.pe, cmd.dst, cmd.src, cmd.size};
        while (extra + 1 < ring_.capacity && extra < 63) {
          rocshmem_proxy_cmd &next = ring_.cmds[(read_ + extra + 1) % ring_.capacity];
          if (__atomic_load_n(&next.valid, __ATOMIC_ACQUIRE) != 1 || next.type != cmd.type) break;
          coalesce::Msg m{next.pe, next.dst, next.src, next.size};
          if (!coalesce::continues(last, m)) break;
          unsigned expect_next = 1;
          if (!__atomic_compare_exchange_n(&next.valid, &expect_next, 2u, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE)) {
            break;   // being cancelled by its producer
          }
          cmd.size += m.size;
          last = m;
          ++extra;
        }
      }
      execute(cmd, seq);
      retire(slot, cmd.status_slot, seq);
      for (unsigned e = 1; e <= extra; ++e) {
        rocshmem_proxy_cmd &next = ring_.cmds[(read_ + e) % ring_.capacity];
        retire(next, next.status_slot, seq + e);
      }
      executed_.fetch_add(1);
      merged_.fetch_add(extra);
      read_ += extra;
    }
    ++read_;
    __atomic_store_n(const_cast<unsigned long long *>(ring_.read_index),
                     static_cast<unsigned long long>(read_), __ATOMIC_RELEASE);
  }
}

void Proxy::retire(volatile rocshmem_proxy_cmd &slot, int status_slot, uint64_t seq) {
  if (status_slot < 0) {
    __atomic_store_n(const_cast<unsigned int *>(&slot.valid), 0u, __ATOMIC_RELEASE);
  } else {
    __atomic_store_n(const_cast<unsigned long long *>(&ring_.status[status_slot]),
                     static_cast<unsigned long long>(seq), __ATOMIC_RELEASE);
  }
}

void Proxy::execute(rocshmem_proxy_cmd &cmd, uint64_t) {
  HostOps &ops = rt_->ops();
  HostCtx *ctx = rt_->default_ctx();
  rt_->count(ROCSHMEM_STAT_PROXY_CMD);
  unsigned long long fetched = 0;
  try {
    // Collective commands name their team by its slot; an unknown slot fails the command.
    HostTeam *team = rt_->team_from_slot(static_cast<int>(cmd.team_slot));
    const bool collective = cmd.type == ROCSHMEM_PROXY_BARRIER || cmd.type == ROCSHMEM_PROXY_BROADCAST ||
                            cmd.type == ROCSHMEM_PROXY_REDUCE || cmd.type == ROCSHMEM_PROXY_FCOLLECT ||
                            cmd.type == ROCSHMEM_PROXY_ALLTOALL;
    if (collective && team == nullptr) {
      fetched = static_cast<unsigned long long>(ROCSHMEM_ERROR);
      if (cmd.status_slot >= 0) {
        __atomic_store_n(const_cast<unsigned long long *>(&ring_.fetched[cmd.status_slot]), fetched,
                         __ATOMIC_RELAXED);
      }
      return;
    }
    switch (cmd.type) {
      case ROCSHMEM_PROXY_PUT:
        ops.put(ctx, reinterpret_cast<void *>(cmd.dst), reinterpret_cast<const void *>(cmd.src),
                cmd.size, cmd.pe, true);
        break;
      case ROCSHMEM_PROXY_GET:
        ops.get(ctx, reinterpret_cast<void *>(cmd.dst), reinterpret_cast<const void *>(cmd.src),
                cmd.size, cmd.pe, true);
        break;
      case ROCSHMEM_PROXY_AMO_FADD:
        fetched = ops.amo(ctx, AmoOp::ADD, dtype_for_size(cmd.dtype_size),
                          reinterpret_cast<void *>(cmd.dst), cmd.size, 0, cmd.pe);
        break;
      case ROCSHMEM_PROXY_AMO_CAS:
        fetched = ops.amo(ctx, AmoOp::CAS, dtype_for_size(cmd.dtype_size),
                          reinterpret_cast<void *>(cmd.dst), cmd.size, cmd.cond, cmd.pe);
        break;
      case ROCSHMEM_PROXY_AMO:
        if (cmd.op > static_cast<unsigned>(AmoOp::XOR)) throw std::invalid_argument("atomic operation code");
        fetched = ops.amo(ctx, static_cast<AmoOp>(cmd.op), dtype_for_size(cmd.dtype_size),
                          reinterpret_cast<void *>(cmd.dst), cmd.size, cmd.cond, cmd.pe);
        break;
      case ROCSHMEM_PROXY_SIGNAL:
        fetched = ops.amo(ctx, cmd.op == ROCSHMEM_SIGNAL_ADD ? AmoOp::ADD : AmoOp::SWAP, DType::U64,
                          reinterpret_cast<void *>(cmd.dst), cmd.size, 0, cmd.pe);
        break;
      case ROCSHMEM_PROXY_QUIET:
        ops.quiet(ctx);
        break;
      case ROCSHMEM_PROXY_BARRIER:
        fetched = static_cast<unsigned long long>(ops.barrier(ctx, team, false));
        break;
      case ROCSHMEM_PROXY_FENCE:
        ops.fence(ctx);
        break;
      case ROCSHMEM_PROXY_P: {
        // The value travels inside the command; stage it in host memory for the put.
        unsigned long long bits = cmd.size;
        ops.put(ctx, reinterpret_cast<void *>(cmd.dst), &bits, cmd.dtype_size, cmd.pe, true);
        break;
      }
      case ROCSHMEM_PROXY_BROADCAST:
        fetched = static_cast<unsigned long long>(ops.broadcast(
            ctx, team, reinterpret_cast<void *>(cmd.dst), reinterpret_cast<const void *>(cmd.src),
            cmd.size, cmd.pe));
        break;
      case ROCSHMEM_PROXY_REDUCE:
        fetched = static_cast<unsigned long long>(ops.reduce(
            ctx, team, reinterpret_cast<void *>(cmd.dst), reinterpret_cast<const void *>(cmd.src),
            cmd.size, static_cast<DType>(cmd.cond), static_cast<ROCSHMEM_OP>(cmd.op)));
        break;
      case ROCSHMEM_PROXY_FCOLLECT:
        fetched = static_cast<unsigned long long>(ops.fcollect(
            ctx, team, reinterpret_cast<void *>(cmd.dst), reinterpret_cast<const void *>(cmd.src), cmd.size));
        break;
      case ROCSHMEM_PROXY_ALLTOALL:
        fetched = static_cast<unsigned long long>(ops.alltoall(
            ctx, team, reinterpret_cast<void *>(cmd.dst), reinterpret_cast<const void *>(cmd.src), cmd.size));
        break;
      default:
        break;
    }
  } catch (const std::exception &) {
    // A malformed command must not take the consumer down; the producer sees no completion.
    return;
  }
  if (cmd.status_slot >= 0) {
    __atomic_store_n(const_cast<unsigned long long *>(&ring_.fetched[cmd.status_slot]), fetched,
                     __ATOMIC_RELAXED);
  }
}

std::string Proxy::describe_command(unsigned index) const {
  static const char *const states[] = {"free", "published", "claimed", "cancelled"};
  static const char *const ops[] = {"nop", "put", "get", "amo_fadd", "amo_cas", "quiet", "barrier", "signal",
                                    "fence", "broadcast", "reduce", "fcollect", "alltoall", "p"};
  if (ring_.cmds == nullptr || ring_.capacity == 0) return "no ring";
  const unsigned i = index & (ring_.capacity - 1);
  const volatile rocshmem_proxy_cmd &c = ring_.cmds[i];
  const unsigned valid = c.valid, type = c.type;
  char line[320];
  std::snprintf(line, sizeof(line),
                "slot %u of %u: %s, op %s (%u), pe %d, dst 0x%llx, src 0x%llx, size %llu, cond %llu, sub-op %u, "
                "element %u bytes, team slot %llu, completion slot %d",
                i, ring_.capacity, valid < 4 ? states[valid] : "corrupt", type < 14 ? ops[type] : "unknown", type, c.pe,
                c.dst, c.src, c.size, c.cond, c.op, c.dtype_size, c.team_slot, c.status_slot);
  return line;
}

std::string Proxy::describe_completion(unsigned index) const {
  if (ring_.status == nullptr || ring_.n_status == 0) return "no ring";
  const unsigned i = index % ring_.n_status;
  char line[200];
  std::snprintf(line, sizeof(line),
                "completion %u of %u: last acknowledged command %llu (0: none yet), fetched value %llu (0x%llx); "
                "consumer has retired %llu commands",
                i, ring_.n_status, static_cast<unsigned long long>(ring_.status[i]),
                static_cast<unsigned long long>(ring_.fetched[i]), static_cast<unsigned long long>(ring_.fetched[i]),
                static_cast<unsigned long long>(ring_.read_index ? *ring_.read_index : 0));
  return line;
}

int Proxy::submit(const rocshmem_proxy_cmd &in, bool blocking, uint64_t *fetched, uint64_t timeout_ms) {
  if (!running_.load()) return ROCSHMEM_ERROR;
  using Clock = std::chrono::steady_clock;
  auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  // Reserve an index only once its slot is known to be free: the ring is not full (the command
  // `capacity` positions earlier has been consumed) and a blocking user of the slot has released
  // it. An index is therefore never taken and then abandoned, which would stall the consumer.
  uint64_t idx;
  unsigned s;
  for (;;) {
    idx = host_write_.load();
    s = static_cast<unsigned>(idx % ring_.capacity);
    uint64_t rd = __atomic_load_n(const_cast<unsigned long long *>(ring_.read_index), __ATOMIC_ACQUIRE);
    if (idx - rd < ring_.capacity && __atomic_load_n(&ring_.cmds[s].valid, __ATOMIC_ACQUIRE) == 0) {
      if (host_write_.compare_exchange_weak(idx, idx + 1)) break;
      continue;
    }
    if (Clock::now() > deadline) return ROCSHMEM_ERROR;
    std::this_thread::yield();
  }
  rocshmem_proxy_cmd &slot = ring_.cmds[s];
  rocshmem_proxy_cmd cmd = in;
  cmd.status_slot = blocking ? static_cast<int>(s) : -1;
  cmd.valid = 0;
  std::memcpy(const_cast<rocshmem_proxy_cmd *>(&slot), &cmd, sizeof(cmd));
  __atomic_store_n(&slot.valid, 1u, __ATOMIC_RELEASE);
  if (!blocking) return ROCSHMEM_SUCCESS;
  int rc = ROCSHMEM_SUCCESS;
  while (__atomic_load_n(const_cast<unsigned long long *>(&ring_.status[s]), __ATOMIC_ACQUIRE) < idx + 1) {
    if (Clock::now() > deadline) {
      rc = ROCSHMEM_ERROR;
      break;
    }
    std::this_thread::yield();
  }
  if (rc == ROCSHMEM_SUCCESS && fetched) {
    *fetched = __atomic_load_n(const_cast<unsigned long long *>(&ring_.fetched[s]), __ATOMIC_RELAXED);
  }
  if (rc != ROCSHMEM_SUCCESS) {
    // Not picked up yet: mark it cancelled and let the consumer retire the slot in order.
    unsigned expected = 1;
    if (__atomic_compare_exchange_n(&slot.valid, &expected, 3u, false, __ATOMIC_ACQ_REL,
                                    __ATOMIC_ACQUIRE)) {
      return rc;
    }
  }
  // The producer of a blocking command releases the slot.
  __atomic_store_n(&slot.valid, 0u, __ATOMIC_RELEASE);
  return rc;
}

}  // namespace rocshmem
