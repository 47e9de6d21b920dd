// Host-API engine for the shared-memory (CPU) heap.
#include <chrono>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

#include "host_ops.hpp"
#include "runtime.hpp"

namespace rocshmem {

size_t dtype_size(DType t) {
  switch (t) {
    case DType::I8: case DType::U8: return 1;
    case DType::I16: case DType::U16: case DType::F16: case DType::BF16: return 2;
    case DType::I32: case DType::U32: case DType::F32: return 4;
    default: return 8;
  }
}
bool dtype_is_float(DType t) {
  return t == DType::F32 || t == DType::F64 || t == DType::F16 || t == DType::BF16;
}
bool dtype_is_signed(DType t) {
  return t == DType::I8 || t == DType::I16 || t == DType::I32 || t == DType::I64 || dtype_is_float(t);
}

namespace {

float half_to_float(uint16_t h) {
  uint32_t sign = (h >> 15) & 1u, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign << 31;
    } else {
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400u));
      bits = (sign << 31) | ((127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    bits = (sign << 31) | 0x7f800000u | (man << 13);
  } else {
    bits = (sign << 31) | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

uint16_t float_to_half(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  int32_t exp = static_cast<int32_t>((x >> 23) & 0xff) - 127 + 15;
  uint32_t man = x & 0x7fffffu;
  if (((x >> 23) & 0xff) == 0xff) return static_cast<uint16_t>(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31) return static_cast<uint16_t>(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return static_cast<uint16_t>(sign);
    man |= 0x800000u;
    uint32_t shift = static_cast<uint32_t>(14 - exp);
    uint32_t half = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    return static_cast<uint16_t>(sign | half);
  }
  uint32_t half = (static_cast<uint32_t>(exp) << 10) | (man >> 13);
  uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
  return static_cast<uint16_t>(sign | half);
}

float bf16_to_float(uint16_t b) {
  uint32_t bits = static_cast<uint32_t>(b) << 16;
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

uint16_t float_to_bf16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((x >> 16) | 0x40);
  uint32_t lsb = (x >> 16) & 1u;
  x += 0x7fffu + lsb;
  return static_cast<uint16_t>(x >> 16);
}

double load_as_double(const void *p, DType t) {
  switch (t) {
    case DType::F32: { float v; std::memcpy(&v, p, 4); return v; }
    case DType::F64: { double v; std::memcpy(&v, p, 8); return v; }
    case DType::F16: { uint16_t v; std::memcpy(&v, p, 2); return half_to_float(v); }
    case DType::BF16: { uint16_t v; std::memcpy(&v, p, 2); return bf16_to_float(v); }
    default: return 0.0;
  }
}

void store_from_double(void *p, DType t, double d) {
  switch (t) {
    case DType::F32: { float v = static_cast<float>(d); std::memcpy(p, &v, 4); break; }
    case DType::F64: std::memcpy(p, &d, 8); break;
    case DType::F16: { uint16_t v = float_to_half(static_cast<float>(d)); std::memcpy(p, &v, 2); break; }
    case DType::BF16: { uint16_t v = float_to_bf16(static_cast<float>(d)); std::memcpy(p, &v, 2); break; }
    default: break;
  }
}

int64_t load_as_i64(const void *p, DType t) {
  switch (t) {
    case DType::I8: { int8_t v; std::memcpy(&v, p, 1); return v; }
    case DType::U8: { uint8_t v; std::memcpy(&v, p, 1); return v; }
    case DType::I16: { int16_t v; std::memcpy(&v, p, 2); return v; }
    case DType::U16: { uint16_t v; std::memcpy(&v, p, 2); return v; }
    case DType::I32: { int32_t v; std::memcpy(&v, p, 4); return v; }
    case DType::U32: { uint32_t v; std::memcpy(&v, p, 4); return v; }
    default: { int64_t v; std::memcpy(&v, p, 8); return v; }
  }
}

template <typename T>
T apply_int(T a, T b, ROCSHMEM_OP op) {
  switch (op) {
    case ROCSHMEM_SUM: return static_cast<T>(a + b);
    case ROCSHMEM_PROD: return static_cast<T>(a * b);
    case ROCSHMEM_MIN: return a < b ? a : b;
    case ROCSHMEM_MAX: return a > b ? a : b;
    case ROCSHMEM_AND: return static_cast<T>(a & b);
    case ROCSHMEM_OR: return static_cast<T>(a | b);
    case ROCSHMEM_XOR: return static_cast<T>(a ^ b);
    default: return b;
  }
}

template <typename T>
void reduce_int(void *acc, const void *in, size_t n, ROCSHMEM_OP op) {
  T *a = static_cast<T *>(acc);
  const T *b = static_cast<const T *>(in);
  for (size_t i = 0; i < n; ++i) a[i] = apply_int<T>(a[i], b[i], op);
}

void reduce_into(void *acc, const void *in, size_t n, DType t, ROCSHMEM_OP op) {
  switch (t) {
    case DType::I8: reduce_int<int8_t>(acc, in, n, op); return;
    case DType::U8: reduce_int<uint8_t>(acc, in, n, op); return;
    case DType::I16: reduce_int<int16_t>(acc, in, n, op); return;
    case DType::U16: reduce_int<uint16_t>(acc, in, n, op); return;
    case DType::I32: reduce_int<int32_t>(acc, in, n, op); return;
    case DType::U32: reduce_int<uint32_t>(acc, in, n, op); return;
    case DType::I64: reduce_int<int64_t>(acc, in, n, op); return;
    case DType::U64: reduce_int<uint64_t>(acc, in, n, op); return;
    default: break;
  }
  size_t sz = dtype_size(t);
  char *a = static_cast<char *>(acc);
  const char *b = static_cast<const char *>(in);
  for (size_t i = 0; i < n; ++i) {
    double x = load_as_double(a + i * sz, t), y = load_as_double(b + i * sz, t), r;
    switch (op) {
      case ROCSHMEM_SUM: r = x + y; break;
      case ROCSHMEM_PROD: r = x * y; break;
      case ROCSHMEM_MIN: r = x < y ? x : y; break;
      case ROCSHMEM_MAX: r = x > y ? x : y; break;
      default: r = y; break;
    }
    store_from_double(a + i * sz, t, r);
  }
}

template <typename T>
uint64_t amo_int(T *p, AmoOp op, uint64_t value, uint64_t cond) {
  T v = static_cast<T>(value), old{};
  switch (op) {
    case AmoOp::FETCH: old = __atomic_load_n(p, __ATOMIC_SEQ_CST); break;
    case AmoOp::SWAP: old = __atomic_exchange_n(p, v, __ATOMIC_SEQ_CST); break;
    case AmoOp::CAS: {
      T expected = static_cast<T>(cond);
      __atomic_compare_exchange_n(p, &expected, v, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST);
      old = expected;
      break;
    }
    case AmoOp::ADD: old = __atomic_fetch_add(p, v, __ATOMIC_SEQ_CST); break;
    case AmoOp::AND: old = __atomic_fetch_and(p, v, __ATOMIC_SEQ_CST); break;
    case AmoOp::OR: old = __atomic_fetch_or(p, v, __ATOMIC_SEQ_CST); break;
    case AmoOp::XOR: old = __atomic_fetch_xor(p, v, __ATOMIC_SEQ_CST); break;
  }
  uint64_t bits = 0;
  std::memcpy(&bits, &old, sizeof(T));
  return bits;
}

template <typename F, typename I>
uint64_t amo_float(I *p, AmoOp op, uint64_t value, uint64_t cond) {
  if (op != AmoOp::ADD) return amo_int<I>(p, op, value, cond);  // fetch/swap/cas act on the bits
  I add_bits = static_cast<I>(value);
  F add;
  std::memcpy(&add, &add_bits, sizeof(F));
  I old = __atomic_load_n(p, __ATOMIC_SEQ_CST);
  for (;;) {
    F cur;
    std::memcpy(&cur, &old, sizeof(F));
    F next = cur + add;
    I next_bits;
    std::memcpy(&next_bits, &next, sizeof(F));
    if (__atomic_compare_exchange_n(p, &old, next_bits, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST)) break;
  }
  return static_cast<uint64_t>(old);
}

uint64_t load_bits(const void *p, DType t) {
  switch (dtype_size(t)) {
    case 1: return __atomic_load_n(static_cast<const uint8_t *>(p), __ATOMIC_ACQUIRE);
    case 2: return __atomic_load_n(static_cast<const uint16_t *>(p), __ATOMIC_ACQUIRE);
    case 4: return __atomic_load_n(static_cast<const uint32_t *>(p), __ATOMIC_ACQUIRE);
    default: return __atomic_load_n(static_cast<const uint64_t *>(p), __ATOMIC_ACQUIRE);
  }
}

class CpuHostOps final : public HostOps {
 public:
  explicit CpuHostOps(Runtime *rt) : rt_(rt) {}

  void put(HostCtx *, void *dst, const void *src, size_t bytes, int pe, bool) override {
    std::memcpy(rt_->translate(dst, pe), src, bytes);
    __atomic_thread_fence(__ATOMIC_RELEASE);
  }
  void get(HostCtx *, void *dst, const void *src, size_t bytes, int pe, bool) override {
    __atomic_thread_fence(__ATOMIC_ACQUIRE);
    std::memcpy(dst, rt_->translate(src, pe), bytes);
  }
  uint64_t amo(HostCtx *, AmoOp op, DType t, void *target, uint64_t value, uint64_t cond,
               int pe) override {
    void *p = rt_->translate(target, pe);
    switch (t) {
      case DType::F32: return amo_float<float, uint32_t>(static_cast<uint32_t *>(p), op, value, cond);
      case DType::F64: return amo_float<double, uint64_t>(static_cast<uint64_t *>(p), op, value, cond);
      default: break;
    }
    switch (dtype_size(t)) {
      case 4: return amo_int<uint32_t>(static_cast<uint32_t *>(p), op, value, cond);
      case 8: return amo_int<uint64_t>(static_cast<uint64_t *>(p), op, value, cond);
      case 2: return amo_int<uint16_t>(static_cast<uint16_t *>(p), op, value, cond);
      default: return amo_int<uint8_t>(static_cast<uint8_t *>(p), op, value, cond);
    }
  }
  void fence(HostCtx *) override { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
  void quiet(HostCtx *) override { __atomic_thread_fence(__ATOMIC_SEQ_CST); }

  int test(void *ivar, DType t, int cmp, uint64_t value) override {
    return compare_bits(load_bits(ivar, t), t, cmp, value) ? 1 : 0;
  }

  int wait_until(void *ivar, DType t, int cmp, uint64_t value) override {
    auto deadline = std::chrono::steady_clock::now() +
                    std::chrono::milliseconds(rt_->config().wait_timeout_ms);
    unsigned spins = 0;
    uint64_t seen = 0;
    for (;;) {
      seen = load_bits(ivar, t);
      if (compare_bits(seen, t, cmp, value)) return ROCSHMEM_SUCCESS;
      if ((++spins & 255u) == 0) {
        if (std::chrono::steady_clock::now() > deadline) break;
        std::this_thread::yield();
      }
    }
    record(ROCSHMEM_ERR_WAIT_TIMEOUT, -1, ivar, value, seen);
    return ROCSHMEM_ERROR;
  }

  // Epoch barrier: every local member publishes its team's next epoch into its slot on every
  // member, then waits until every member's slot in its own array has reached that epoch.
  int barrier(HostCtx *, HostTeam *team, bool) override {
    __atomic_thread_fence(__ATOMIC_SEQ_CST);
    const auto &lay = rt_->layout();
    const int n = team->world.size;
    std::vector<unsigned long long> epoch(rt_->n_local(), 0);
    for (int l = 0; l < rt_->n_local(); ++l) {
      int me = team->my_pe[l];
      if (me < 0) continue;
      int my_world = rt_->first_pe() + l;
      auto *td = reinterpret_cast<rocshmem_team_dev *>(rt_->internal_base(my_world) + lay.teams) + team->slot;
      epoch[l] = ++td->barrier_epoch;
      for (int j = 0; j < n; ++j) {
        int w = team->world.pe_in_world(j);
        auto *flags = reinterpret_cast<unsigned long long *>(rt_->internal_base(w) + lay.barrier_flags);
        __atomic_store_n(&flags[size_t(team->slot) * ROCSHMEM_MAX_PES + me], epoch[l], __ATOMIC_RELEASE);
      }
    }
    auto deadline = std::chrono::steady_clock::now() +
                    std::chrono::milliseconds(rt_->config().wait_timeout_ms);
    for (int l = 0; l < rt_->n_local(); ++l) {
      if (team->my_pe[l] < 0) continue;
      int my_world = rt_->first_pe() + l;
      auto *flags = reinterpret_cast<unsigned long long *>(rt_->internal_base(my_world) + lay.barrier_flags);
      for (int j = 0; j < n; ++j) {
        unsigned long long *f = &flags[size_t(team->slot) * ROCSHMEM_MAX_PES + j];
        unsigned spins = 0;
        while (__atomic_load_n(f, __ATOMIC_ACQUIRE) < epoch[l]) {
          if ((++spins & 255u) == 0) {
            if (std::chrono::steady_clock::now() > deadline) {
              record(ROCSHMEM_ERR_BARRIER_TIMEOUT, team->world.pe_in_world(j), f, epoch[l],
                     __atomic_load_n(f, __ATOMIC_ACQUIRE));
              return ROCSHMEM_ERROR;
            }
            std::this_thread::yield();
          }
        }
      }
    }
    return ROCSHMEM_SUCCESS;
  }

  int broadcast(HostCtx *ctx, HostTeam *team, void *dst, const void *src, size_t bytes,
                int root) override {
    if (barrier(ctx, team, true) != ROCSHMEM_SUCCESS) return ROCSHMEM_ERROR;
    int root_world = team->world.pe_in_world(root);
    for (int l = 0; l < rt_->n_local(); ++l) {
      int me = team->my_pe[l];
      if (me < 0 || me == root) continue;  // the root's dest is left untouched
      int my_world = rt_->first_pe() + l;
      std::memcpy(rt_->translate(dst, my_world), rt_->translate(src, root_world), bytes);
    }
    return barrier(ctx, team, true);
  }

  int reduce(HostCtx *ctx, HostTeam *team, void *dst, const void *src, size_t nelems, DType t,
             ROCSHMEM_OP op) override {
    if (barrier(ctx, team, true) != ROCSHMEM_SUCCESS) return ROCSHMEM_ERROR;
    size_t bytes = nelems * dtype_size(t);
    std::vector<std::vector<char>> results(rt_->n_local());
    for (int l = 0; l < rt_->n_local(); ++l) {
      if (team->my_pe[l] < 0) continue;
      auto &acc = results[l];
      acc.resize(bytes);
      std::memcpy(acc.data(), rt_->translate(src, team->world.pe_in_world(0)), bytes);
      for (int j = 1; j < team->world.size; ++j) {
        reduce_into(acc.data(), rt_->translate(src, team->world.pe_in_world(j)), nelems, t, op);
      }
    }
    // Sources may alias destinations: nobody writes before everybody has finished reading.
    if (barrier(ctx, team, true) != ROCSHMEM_SUCCESS) return ROCSHMEM_ERROR;
    for (int l = 0; l < rt_->n_local(); ++l) {
      if (team->my_pe[l] < 0) continue;
      std::memcpy(rt_->translate(dst, rt_->first_pe() + l), results[l].data(), bytes);
    }
    return barrier(ctx, team, true);
  }

  int fcollect(HostCtx *ctx, HostTeam *team, void *dst, const void *src, size_t bytes) override {
    if (barrier(ctx, team, true) != ROCSHMEM_SUCCESS) return ROCSHMEM_ERROR;
    for (int l = 0; l < rt_->n_local(); ++l) {
      if (team->my_pe[l] < 0) continue;
      char *d = static_cast<char *>(rt_->translate(dst, rt_->first_pe() + l));
      for (int j = 0; j < team->world.size; ++j) {
        std::memcpy(d + size_t(j) * bytes, rt_->translate(src, team->world.pe_in_world(j)), bytes);
      }
    }
    return barrier(ctx, team, true);
  }

  int alltoall(HostCtx *ctx, HostTeam *team, void *dst, const void *src, size_t bytes) override {
    if (barrier(ctx, team, true) != ROCSHMEM_SUCCESS) return ROCSHMEM_ERROR;
    for (int l = 0; l < rt_->n_local(); ++l) {
      int me = team->my_pe[l];
      if (me < 0) continue;
      char *d = static_cast<char *>(rt_->translate(dst, rt_->first_pe() + l));
      for (int j = 0; j < team->world.size; ++j) {
        const char *s = static_cast<const char *>(rt_->translate(src, team->world.pe_in_world(j)));
        std::memcpy(d + size_t(j) * bytes, s + size_t(me) * bytes, bytes);
      }
    }
    return barrier(ctx, team, true);
  }

  void ctx_init(HostCtx *) override {}
  void ctx_fini(HostCtx *) override {}

 private:
  void record(uint32_t kind, int pe, const void *addr, uint64_t expected, uint64_t observed) {
    int my_world = rt_->my_pe();
    auto *e = reinterpret_cast<rocshmem_error_record *>(rt_->internal_base(my_world) + rt_->layout().error);
    if (__atomic_fetch_add(&e->count, 1u, __ATOMIC_SEQ_CST) == 0) {
      e->kind = kind;
      e->pe = pe;
      e->where = 0;
      e->addr = reinterpret_cast<uint64_t>(addr);
      e->expected = expected;
      e->observed = observed;
    }
    rt_->count(ROCSHMEM_STAT_TIMEOUTS);
  }
  Runtime *rt_;
};

}  // namespace

bool compare_bits(uint64_t observed, DType t, int cmp, uint64_t value) {
  auto decide = [cmp](auto a, auto b) {
    switch (cmp) {
      case ROCSHMEM_CMP_EQ: return a == b;
      case ROCSHMEM_CMP_NE: return a != b;
      case ROCSHMEM_CMP_GT: return a > b;
      case ROCSHMEM_CMP_GE: return a >= b;
      case ROCSHMEM_CMP_LT: return a < b;
      case ROCSHMEM_CMP_LE: return a <= b;
      default: return false;
    }
  };
  if (dtype_is_float(t)) return decide(load_as_double(&observed, t), load_as_double(&value, t));
  if (dtype_is_signed(t)) return decide(load_as_i64(&observed, t), load_as_i64(&value, t));
  uint64_t mask = dtype_size(t) == 8 ? ~uint64_t(0) : ((uint64_t(1) << (8 * dtype_size(t))) - 1);
  return decide(observed & mask, value & mask);
}

HostOps *make_cpu_host_ops(Runtime *rt) { return new CpuHostOps(rt); }

}  // namespace rocshmem
