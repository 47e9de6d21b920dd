// Tensor-parallel GEMMs fused with their collective, on heap-resident operands (one PE per process).
//
// all-gather -> GEMM (ag_gemm_bf16): one kernel. Every CTA runs the tcgen05 GEMM core plus one extra
// "push" warp. The push warps of a rank store that rank's activation shard into the gathered buffer of
// every member (16-byte peer stores over NVLink, destinations in the order in which they will need the
// rows), slice by slice, and bump a per-row-block counter on the receiver after each slice. The GEMM
// roles walk the row blocks in arrival order (local shard first); the TMA producer of a CTA waits for
// its row block's counter before loading A. The transfer of later row blocks overlaps the math on
// earlier ones, and remote rows cross NVLink once (every CTA then reads them from local HBM / L2).
//
// GEMM -> reduce-scatter (gemm_rs_bf16): the GEMM epilogue stores each finished tile straight into the
// staging buffer of the rank that owns those rows (16-byte peer stores), tiles ordered so that the ranks
// write to different owners at any time and a rank's own rows come last. After a grid barrier and a
// cross-rank barrier every CTA sums its share of the n_ranks staged partials of the local rows in fp32
// and writes the bf16 result. (A form that added the partials in the epilogue of the owner's tiles, with
// one arrival counter per tile and no reduction pass, was measured and removed: the owner's tiles are the
// last 1 / n of the kernel and four epilogue warps per SM cannot pull n - 1 partial tiles fast enough, so
// the reduce-scatter alone took 541 us against 409 us on eight GPUs.)
//
// Nothing here has a counterpart in the reference; the ingredients it offers are fcollect, reduction
// and put-with-signal (src/ipc/context_ipc_tmpl_device.hpp:166-531).
#include <cuda.h>

#include <cstdlib>
#include <cuda_bf16.h>

#include "gemm_core.cuh"
#include "gemm2_core.cuh"
#include "gemm_fp8_core.cuh"
#include "gemm_kernels.hpp"
#include "gemm_tmap.hpp"
#include "launch.cuh"
#include "lib_common.cuh"

namespace rocshmem {
namespace kernels {

namespace {

using detail::remote_ptr;
using detail::team_pe_to_world;

constexpr int kPushSlice = 16 * 1024;  // bytes one push warp moves to one destination between two flags

// What the push warps move: row blocks of 128 rows of this rank's shard (`src`, local) into every
// member's `dst` (symmetric; block b of member s lands at block s * tiles_per_shard + b), optionally
// with a second, smaller array (the rows' fp8 scales). Pushing (stores) instead of pulling (loads)
// matters: a store needs no round trip, so one warp per SM keeps NVLink busy, while remote loads need
// thousands of threads in flight.
struct AgPush {
  const rocshmem_team_dev *team;
  const char *src;
  char *dst;
  size_t tile_bytes;   // multiple of 16
  const char *src2;
  char *dst2;
  size_t tile2_bytes;  // 0: none
  int tiles_per_shard;
  unsigned int *ready;  // symmetric [n_ranks * tiles_per_shard], monotonic: += slices per row block and call
};

__device__ __forceinline__ int ag_slices_per_tile(size_t tile_bytes) {
  return static_cast<int>((tile_bytes + kPushSlice - 1) / kPushSlice);
}

// One warp: copies `bytes` (multiple of 16) with up to eight 16-byte loads in flight per lane.
__device__ __forceinline__ void warp_copy16(char *dst, const char *src, size_t bytes, int lane) {
  const size_t nvec = bytes / 16;
  size_t v = lane;
  for (; v + 7 * 32 < nvec; v += 8 * 32) {
    int4 r[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = reinterpret_cast<const int4 *>(src)[v + i * 32];
#pragma unroll
    for (int i = 0; i < 8; ++i) reinterpret_cast<int4 *>(dst)[v + i * 32] = r[i];
  }
  for (; v < nvec; v += 32) reinterpret_cast<int4 *>(dst)[v] = reinterpret_cast<const int4 *>(src)[v];
}

// Run by one extra warp of every CTA. Destinations are served in the order in which they need this
// rank's rows (the rank itself first, then the rank that consumes them second, ...); within a destination
// the (row block, slice) pairs are dealt round-robin to the CTAs. After a slice has been stored and
// fenced, the receiver's counter of that row block is bumped with a release-ordered remote reduction.
__device__ void ag_push_role(const AgPush &a) {
  const rocshmem_team_dev *t = a.team;
  const int lane = threadIdx.x % 32;
  const int P = t->size, me = t->my_pe;
  const int spt = ag_slices_per_tile(a.tile_bytes);
  const long per_dest = long(a.tiles_per_shard) * spt;
  const long total = long(P) * per_dest;
  for (long j = blockIdx.x; j < total; j += gridDim.x) {
    const int d = int(j / per_dest);
    const long rem = j % per_dest;
    const int mt = int(rem / spt), sl = int(rem % spt);
    const int dest = (me - d + P) % P;
    const int world_pe = team_pe_to_world(t, dest);
    const size_t dst_tile = size_t(me) * a.tiles_per_shard + mt;
    const size_t off = size_t(sl) * kPushSlice;
    const size_t left = a.tile_bytes - off;
    warp_copy16(remote_ptr(a.dst + dst_tile * a.tile_bytes + off, world_pe), a.src + size_t(mt) * a.tile_bytes + off,
                left < size_t(kPushSlice) ? left : size_t(kPushSlice), lane);
    if (a.tile2_bytes != 0 && sl == 0) {
      warp_copy16(remote_ptr(a.dst2 + dst_tile * a.tile2_bytes, world_pe), a.src2 + size_t(mt) * a.tile2_bytes,
                  a.tile2_bytes, lane);
    }
    __threadfence_system();  // every lane's stores are ordered before the flag update below
    __syncwarp();
    if (lane == 0) {
      // Row block index at the receiver, in its arrival order: this rank is its d-th source.
      unsigned int *flag = remote_ptr(a.ready + size_t(d) * a.tiles_per_shard + mt, world_pe);
      asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(flag), "r"(1u) : "memory");
    }
  }
}

struct AgArgs {
  rocshmem_team_t team;
  const __nv_bfloat16 *x_shard;   // local or symmetric [m_shard, k]: only read by its owner
  __nv_bfloat16 *gathered;        // symmetric [n_ranks * m_shard, k]: written by every member
  unsigned int *ready;            // symmetric [n_ranks * m_shard / 128], monotonic
  __nv_bfloat16 *c;
  int m_shard, n, k;
  unsigned epoch;
};

// With SWIGLU the weight holds gate rows [0, n / 2) and up rows [n / 2, n); one tile pairs 128 gate
// columns with the matching up columns and the output is silu(gate) * up of width n / 2.
template <bool SWIGLU>
struct AgScheduler {
  int me, n_ranks, tiles_per_shard, tiles_n, tiles, m_shard, n;
  const unsigned int *ready_count;
  unsigned target;
  AgPush push;
  __device__ bool get(int iter, gemm::Tile &t) const {
    const int id = blockIdx.x + iter * gridDim.x;
    if (id >= tiles) return false;
    int oi, nt;  // oi: row block in arrival order
    gemm::raster(id, tiles / tiles_n, tiles_n, min(gemm::RASTER_GROUP, tiles_per_shard), oi, nt);
    const int src = (me + oi / tiles_per_shard) % n_ranks;   // the local shard comes first
    const int mt = oi % tiles_per_shard;
    t.a_row = src * m_shard + mt * gemm::BM;
    t.rows = gemm::BM;
    if (SWIGLU) {
      const int j0 = nt * (gemm::BN / 2);
      t.b_row[0] = j0;
      t.b_row[1] = n / 2 + j0;
      t.cols = min(gemm::BN / 2, n / 2 - j0);
      t.c_col = j0;
    } else {
      t.b_row[0] = nt * gemm::BN;
      t.b_row[1] = nt * gemm::BN + gemm::BN / 2;
      t.cols = min(gemm::BN, n - nt * gemm::BN);
      t.c_col = nt * gemm::BN;
    }
    t.c_row = t.a_row;
    t.tag = oi;
    return true;
  }
  // Called by the TMA producer thread: the row block must have landed in the gathered buffer.
  __device__ bool ready(const gemm::Tile &t) const {
    const unsigned int *p = ready_count + t.tag;
    if (detail::ld_acquire_sys_u32(p) < target) {
      detail::SpinBudget budget(gemm::WAIT_BUDGET_NS);
      while (detail::ld_acquire_sys_u32(p) < target) {
        if (!budget.keep_going()) {
          detail::record_error(ROCSHMEM_ERR_KERNEL, -1, 80, p, target, *reinterpret_cast<const volatile unsigned int *>(p));
          return false;
        }
      }
    }
    sm100::fence_proxy_async();  // the rows were written with generic stores and are read by TMA
    return true;
  }
  __device__ void side_role() const { ag_push_role(push); }
};

struct PlainEpilogue {
  __nv_bfloat16 *c;
  size_t ldc;
  __device__ __nv_bfloat16 *row_ptr(const gemm::Tile &t, int row) const {
    return c + static_cast<size_t>(t.c_row + row) * ldc + t.c_col;
  }
};

template <bool SWIGLU>
__global__ void __launch_bounds__(gemm::THREADS + 32, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, AgArgs a) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm::Shared sh;
  const rocshmem_team_dev *t = detail::team_of(a.team);
  if (t->my_pe < 0) return;
  // Every member has entered this call, so its previous one no longer reads its gathered buffer.
  if (!block_pair_barrier(t, blockIdx.x, false)) return;
  AgScheduler<SWIGLU> sched;
  sched.me = t->my_pe;
  sched.n_ranks = t->size;
  sched.tiles_per_shard = a.m_shard / gemm::BM;
  sched.tiles_n = SWIGLU ? (a.n / 2 + gemm::BN / 2 - 1) / (gemm::BN / 2) : (a.n + gemm::BN - 1) / gemm::BN;
  sched.tiles = t->size * sched.tiles_per_shard * sched.tiles_n;
  sched.m_shard = a.m_shard;
  sched.n = a.n;
  sched.ready_count = a.ready;
  const size_t tile_bytes = size_t(gemm::BM) * a.k * 2;
  sched.target = a.epoch * static_cast<unsigned>(ag_slices_per_tile(tile_bytes));
  sched.push = AgPush{t, reinterpret_cast<const char *>(a.x_shard), reinterpret_cast<char *>(a.gathered), tile_bytes,
                      nullptr, nullptr, 0, a.m_shard / gemm::BM, a.ready};
  PlainEpilogue epi{a.c, static_cast<size_t>(SWIGLU ? a.n / 2 : a.n)};
  gemm::run<false, SWIGLU>(&map_a, &map_b, a.k * 2, sched, epi, smem_raw, sh);
}

// Two-CTA form: a pair of CTAs computes 256 x 256 tiles, i.e. two 128-row blocks of the gathered matrix at
// a time (m_shard must be a multiple of 256); the producer waits for both blocks' counters.
template <bool SWIGLU>
struct AgPairScheduler {
  int me, n_ranks, tiles_per_shard, tiles_n, tiles, m_shard, n;   // tiles_per_shard counts 256-row blocks
  const unsigned int *ready_count;
  unsigned target;
  AgPush push;
  __device__ bool get(int iter, gemm::Tile &t) const {
    const int id = blockIdx.x / 2 + iter * (gridDim.x / 2);
    if (id >= tiles) return false;
    int oi, nt;
    gemm::raster(id, tiles / tiles_n, tiles_n, min(gemm::RASTER_GROUP / 2, tiles_per_shard), oi, nt);
    const int src = (me + oi / tiles_per_shard) % n_ranks;
    const int mt = oi % tiles_per_shard;
    t.a_row = src * m_shard + mt * 2 * gemm2::BM;
    t.rows = 2 * gemm2::BM;
    if (SWIGLU) {
      const int j0 = nt * (gemm2::BN / 2);
      t.b_row[0] = j0;
      t.b_row[1] = n / 2 + j0;
      t.cols = min(gemm2::BN / 2, n / 2 - j0);
      t.c_col = j0;
    } else {
      t.b_row[0] = nt * gemm2::BN;
      t.b_row[1] = nt * gemm2::BN + gemm2::BN / 2;
      t.cols = min(gemm2::BN, n - nt * gemm2::BN);
      t.c_col = nt * gemm2::BN;
    }
    t.c_row = t.a_row;
    t.tag = 2 * oi;   // first of the two 128-row blocks, in arrival order
    return true;
  }
  __device__ bool wait_block(const unsigned int *p) const {
    if (detail::ld_acquire_sys_u32(p) < target) {
      detail::SpinBudget budget(gemm::WAIT_BUDGET_NS);
      while (detail::ld_acquire_sys_u32(p) < target) {
        if (!budget.keep_going()) {
          detail::record_error(ROCSHMEM_ERR_KERNEL, -1, 81, p, target, *reinterpret_cast<const volatile unsigned int *>(p));
          return false;
        }
      }
    }
    return true;
  }
  __device__ bool ready(const gemm::Tile &t) const {
    // Each CTA of the pair loads one of the two row blocks; waiting for both keeps the logic symmetric.
    if (!wait_block(ready_count + t.tag) || !wait_block(ready_count + t.tag + 1)) return false;
    sm100::fence_proxy_async();
    return true;
  }
  __device__ void side_role() const { ag_push_role(push); }
};

template <bool SWIGLU>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(gemm2::THREADS + 32, 1)
ag_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, AgArgs a) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm2::Shared sh;
  const rocshmem_team_dev *t = detail::team_of(a.team);
  if (t->my_pe < 0) return;
  if (!block_pair_barrier(t, blockIdx.x, false)) return;
  AgPairScheduler<SWIGLU> sched;
  sched.me = t->my_pe;
  sched.n_ranks = t->size;
  sched.tiles_per_shard = a.m_shard / (2 * gemm2::BM);
  sched.tiles_n = SWIGLU ? (a.n / 2 + gemm2::BN / 2 - 1) / (gemm2::BN / 2) : (a.n + gemm2::BN - 1) / gemm2::BN;
  sched.tiles = t->size * sched.tiles_per_shard * sched.tiles_n;
  sched.m_shard = a.m_shard;
  sched.n = a.n;
  sched.ready_count = a.ready;
  const size_t tile_bytes = size_t(gemm::BM) * a.k * 2;
  sched.target = a.epoch * static_cast<unsigned>(ag_slices_per_tile(tile_bytes));
  sched.push = AgPush{t, reinterpret_cast<const char *>(a.x_shard), reinterpret_cast<char *>(a.gathered), tile_bytes,
                      nullptr, nullptr, 0, a.m_shard / gemm::BM, a.ready};
  PlainEpilogue epi{a.c, static_cast<size_t>(SWIGLU ? a.n / 2 : a.n)};
  gemm2::run<SWIGLU>(&map_a, &map_b, a.k * 2, sched, epi, smem_raw, sh);
}

// ---- GEMM -> reduce-scatter ----------------------------------------------------------------------------------

struct RsArgs {
  rocshmem_team_t team;
  __nv_bfloat16 *staging;  // symmetric [n_ranks][m_shard, n]: slice s holds rank s's partial of my rows
  __nv_bfloat16 *out;      // local [m_shard, n]
  int m_shard, n, k;
  unsigned long long *grid_counter;
  unsigned epoch;
};

struct RsScheduler {
  int me, n_ranks, tiles_per_shard, tiles_n, tiles, m_shard, n;
  __device__ bool get(int iter, gemm::Tile &t) const {
    const int id = blockIdx.x + iter * gridDim.x;
    if (id >= tiles) return false;
    int oi, nt;
    gemm::raster(id, tiles / tiles_n, tiles_n, min(gemm::RASTER_GROUP, tiles_per_shard), oi, nt);
    // Rows owned by the next rank first, my own rows last: at any time the ranks store to
    // different owners, and the tiles that need no transfer finish the kernel.
    const int owner = (me + 1 + oi / tiles_per_shard) % n_ranks;
    const int mt = oi % tiles_per_shard;
    t.a_row = owner * m_shard + mt * gemm::BM;
    t.rows = gemm::BM;
    t.b_row[0] = nt * gemm::BN;
    t.b_row[1] = nt * gemm::BN + gemm::BN / 2;
    t.cols = min(gemm::BN, n - nt * gemm::BN);
    t.c_row = mt * gemm::BM;   // row inside the owner's shard
    t.c_col = nt * gemm::BN;
    t.tag = owner;
    return true;
  }
  __device__ bool ready(const gemm::Tile &) const { return true; }
  __device__ void side_role() const {}
};

// Tiles go into the owners' staging slices (my own rows into my slice of my own staging buffer).
struct RsEpilogue {
  const rocshmem_team_dev *team;
  __nv_bfloat16 *staging;
  int me, m_shard, n;
  __device__ __nv_bfloat16 *row_ptr(const gemm::Tile &t, int row) const {
    __nv_bfloat16 *local = staging + (static_cast<size_t>(me) * m_shard + t.c_row + row) * n + t.c_col;
    return remote_ptr(local, team_pe_to_world(team, t.tag));
  }
};

// Second half of GEMM -> reduce-scatter, run by every CTA after its tiles are stored.
__device__ void rs_reduce(const RsArgs &a, const rocshmem_team_dev *t) {
  // All CTAs of this rank have stored their tiles (grid barrier), then all ranks have (block b pairs
  // with block b of every peer, which has itself passed its rank's grid barrier): every partial of
  // my rows is in my staging buffers.
  if (!grid_barrier(a.grid_counter, a.epoch, gridDim.x)) return;
  if (!block_pair_barrier(t, blockIdx.x)) return;
  // Sum the n_ranks partials of my rows: 16 bytes per thread and source, all sources in flight.
  const int P = t->size;
  const size_t nvec = static_cast<size_t>(a.m_shard) * a.n / 8;
  const size_t slice = static_cast<size_t>(a.m_shard) * a.n;
  for (size_t v = size_t(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec; v += size_t(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int s0 = 0; s0 < P; s0 += 8) {
      int4 raw[8];
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        if (s0 + s < P) raw[s] = reinterpret_cast<const int4 *>(a.staging + size_t(s0 + s) * slice)[v];
      }
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        if (s0 + s < P) {
          const __nv_bfloat162 *p2 = reinterpret_cast<const __nv_bfloat162 *>(&raw[s]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(p2[i]);
            acc[2 * i] += f.x;
            acc[2 * i + 1] += f.y;
          }
        }
      }
    }
    int4 o;
    __nv_bfloat162 *o2 = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    reinterpret_cast<int4 *>(a.out)[v] = o;
  }
  // The next call stores tiles into the staging buffers as soon as it starts, so nobody leaves
  // before every rank has finished reading its staged partials.
  block_pair_barrier(t, blockIdx.x, false);
}

__global__ void __launch_bounds__(gemm::THREADS, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, RsArgs a) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm::Shared sh;
  const rocshmem_team_dev *t = detail::team_of(a.team);
  if (t->my_pe < 0) return;
  RsScheduler sched;
  sched.me = t->my_pe;
  sched.n_ranks = t->size;
  sched.tiles_per_shard = a.m_shard / gemm::BM;
  sched.tiles_n = (a.n + gemm::BN - 1) / gemm::BN;
  sched.tiles = t->size * sched.tiles_per_shard * sched.tiles_n;
  sched.m_shard = a.m_shard;
  sched.n = a.n;
  RsEpilogue epi{t, a.staging, t->my_pe, a.m_shard, a.n};
  gemm::run<false, false>(&map_a, &map_b, a.k * 2, sched, epi, smem_raw, sh);
  rs_reduce(a, t);
}

struct RsPairScheduler {
  int me, n_ranks, tiles_per_shard, tiles_n, tiles, m_shard, n;   // tiles_per_shard counts 256-row blocks
  __device__ bool get(int iter, gemm::Tile &t) const {
    const int id = blockIdx.x / 2 + iter * (gridDim.x / 2);
    if (id >= tiles) return false;
    int oi, nt;
    gemm::raster(id, tiles / tiles_n, tiles_n, min(gemm::RASTER_GROUP / 2, tiles_per_shard), oi, nt);
    const int owner = (me + 1 + oi / tiles_per_shard) % n_ranks;
    const int mt = oi % tiles_per_shard;
    t.a_row = owner * m_shard + mt * 2 * gemm2::BM;
    t.rows = 2 * gemm2::BM;
    t.b_row[0] = nt * gemm2::BN;
    t.b_row[1] = nt * gemm2::BN + gemm2::BN / 2;
    t.cols = min(gemm2::BN, n - nt * gemm2::BN);
    t.c_row = mt * 2 * gemm2::BM;
    t.c_col = nt * gemm2::BN;
    t.tag = owner;
    return true;
  }
  __device__ bool ready(const gemm::Tile &) const { return true; }
  __device__ void side_role() const {}
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(gemm2::THREADS, 1)
gemm_rs_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, RsArgs a) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm2::Shared sh;
  const rocshmem_team_dev *t = detail::team_of(a.team);
  if (t->my_pe < 0) return;
  RsPairScheduler sched;
  sched.me = t->my_pe;
  sched.n_ranks = t->size;
  sched.tiles_per_shard = a.m_shard / (2 * gemm2::BM);
  sched.tiles_n = (a.n + gemm2::BN - 1) / gemm2::BN;
  sched.tiles = t->size * sched.tiles_per_shard * sched.tiles_n;
  sched.m_shard = a.m_shard;
  sched.n = a.n;
  RsEpilogue epi{t, a.staging, t->my_pe, a.m_shard, a.n};
  gemm2::run<false>(&map_a, &map_b, a.k * 2, sched, epi, smem_raw, sh);
  rs_reduce(a, t);
}

// Kernels with two CTAs per tile are used where the shapes allow; ROCSHMEM_GEMM_TWO_CTA=0 selects the
// one-CTA kernels everywhere (for comparison).
bool use_two_cta() {
  static const bool on = [] {
    const char *e = std::getenv("ROCSHMEM_GEMM_TWO_CTA");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}


// ---- block-scaled e4m3 variants -------------------------------------------------------------------------------
// Same structure with the fp8 core: the push warps send the e4m3 rows and, as a second array, their
// 1 x 128 scales (half the NVLink bytes of the bf16 kernel); the weights carry 128 x 128 scales.

struct Ag8Args {
  rocshmem_team_t team;
  const unsigned char *x_q;   // [m_shard, k] e4m3, read by its owner only
  const float *x_s;           // [m_shard, k / 128]
  unsigned char *gathered_q;  // symmetric [n_ranks * m_shard, k]
  float *gathered_s;          // symmetric [n_ranks * m_shard, k / 128]
  unsigned int *ready;        // symmetric
  const float *b_scale;
  __nv_bfloat16 *c;
  int m_shard, n, k;
  unsigned epoch;
};

template <bool SWIGLU>
__global__ void __launch_bounds__(gemm8::THREADS + 32, 1)
ag_gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, Ag8Args a) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm8::Shared sh;
  const rocshmem_team_dev *t = detail::team_of(a.team);
  if (t->my_pe < 0) return;
  if (!block_pair_barrier(t, blockIdx.x, false)) return;
  AgScheduler<SWIGLU> sched;
  sched.me = t->my_pe;
  sched.n_ranks = t->size;
  sched.tiles_per_shard = a.m_shard / gemm8::BM;
  sched.tiles_n = SWIGLU ? (a.n / 2 + gemm8::BN / 2 - 1) / (gemm8::BN / 2) : (a.n + gemm8::BN - 1) / gemm8::BN;
  sched.tiles = t->size * sched.tiles_per_shard * sched.tiles_n;
  sched.m_shard = a.m_shard;
  sched.n = a.n;
  sched.ready_count = a.ready;
  const size_t tile_bytes = size_t(gemm8::BM) * a.k;
  sched.target = a.epoch * static_cast<unsigned>(ag_slices_per_tile(tile_bytes));
  sched.push = AgPush{t, reinterpret_cast<const char *>(a.x_q), reinterpret_cast<char *>(a.gathered_q), tile_bytes,
                      reinterpret_cast<const char *>(a.x_s), reinterpret_cast<char *>(a.gathered_s),
                      size_t(gemm8::BM) * (a.k / 128) * sizeof(float), a.m_shard / gemm8::BM, a.ready};
  PlainEpilogue epi{a.c, static_cast<size_t>(SWIGLU ? a.n / 2 : a.n)};
  gemm8::run<SWIGLU, true>(&map_a, &map_b, a.gathered_s, a.b_scale, a.k / gemm8::KB, sched, epi, smem_raw, sh);
}

__global__ void __launch_bounds__(gemm8::THREADS, 1)
gemm_rs_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const float *a_scale, const float *b_scale, RsArgs a) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm8::Shared sh;
  const rocshmem_team_dev *t = detail::team_of(a.team);
  if (t->my_pe < 0) return;
  RsScheduler sched;
  sched.me = t->my_pe;
  sched.n_ranks = t->size;
  sched.tiles_per_shard = a.m_shard / gemm8::BM;
  sched.tiles_n = (a.n + gemm8::BN - 1) / gemm8::BN;
  sched.tiles = t->size * sched.tiles_per_shard * sched.tiles_n;
  sched.m_shard = a.m_shard;
  sched.n = a.n;
  RsEpilogue epi{t, a.staging, t->my_pe, a.m_shard, a.n};
  gemm8::run<false, false>(&map_a, &map_b, a_scale, b_scale, a.k / gemm8::KB, sched, epi, smem_raw, sh);
  rs_reduce(a, t);
}

template <typename K>
int prepare_smem(K kernel) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm::SMEM_BYTES);
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // namespace

int fused_error_count() {
  unsigned int v = 0;
  if (cudaMemcpyFromSymbol(&v, gemm::g_gemm_errors, sizeof(v)) != cudaSuccess) return -1;
  return static_cast<int>(v);
}

int ag_gemm_bf16(rocshmem_team_t team, const void *x_shard, void *gathered, unsigned long long *flags,
                 const void *b, void *c, int m_shard, int n, int k, unsigned epoch, int swiglu, void *stream) {
  Runtime &rt = Runtime::instance();
  HostTeam *ht = rt.team_from_handle(team);
  if (!ht || rt.n_local() != 1) return cudaErrorInvalidValue;
  const int P = ht->world.size;
  if (m_shard <= 0 || m_shard % gemm::BM || n <= 0 || n % 8 || k <= 0 || k % 8) return cudaErrorInvalidValue;
  if (swiglu && (n % 16) != 0) return cudaErrorInvalidValue;
  CUtensorMap map_a, map_b;
  if (!encode_tmap_2d(&map_a, gathered, uint64_t(P) * m_shard, k, 2, gemm::BM) ||
      !encode_tmap_2d(&map_b, b, n, k, 2, gemm::BN / 2)) {
    return -1;
  }
  AgArgs a{team, static_cast<const __nv_bfloat16 *>(x_shard), static_cast<__nv_bfloat16 *>(gathered),
           reinterpret_cast<unsigned int *>(flags), static_cast<__nv_bfloat16 *>(c), m_shard, n, k, epoch};
  // The GEMM roles wait for rows that other ranks' CTAs push: all CTAs of all ranks must be resident.
  const int sms = device_sm_count();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (use_two_cta() && m_shard % (2 * gemm2::BM) == 0 && sms % 2 == 0) {
    auto kp = swiglu ? ag_gemm_pair_kernel<true> : ag_gemm_pair_kernel<false>;
    cudaError_t e = cudaFuncSetAttribute(kp, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm2::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    return launch_pes(kp, sms, gemm2::THREADS + 32, gemm2::SMEM_BYTES, s, true, map_a, map_b, a);
  }
  if (int rc = swiglu ? prepare_smem(ag_gemm_kernel<true>) : prepare_smem(ag_gemm_kernel<false>)) return rc;
  if (swiglu) return launch_pes(ag_gemm_kernel<true>, sms, gemm::THREADS + 32, gemm::SMEM_BYTES, s, true, map_a, map_b, a);
  return launch_pes(ag_gemm_kernel<false>, sms, gemm::THREADS + 32, gemm::SMEM_BYTES, s, true, map_a, map_b, a);
}

int gemm_rs_bf16(rocshmem_team_t team, const void *a_mat, const void *b, void *staging, void *out, int m_shard,
                 int n, int k, unsigned long long *grid_counter, unsigned epoch, void *stream) {
  Runtime &rt = Runtime::instance();
  HostTeam *ht = rt.team_from_handle(team);
  if (!ht || rt.n_local() != 1) return cudaErrorInvalidValue;
  const int P = ht->world.size;
  if (m_shard <= 0 || m_shard % gemm::BM || n <= 0 || n % 8 || k <= 0 || k % 8) return cudaErrorInvalidValue;
  CUtensorMap map_a, map_b;
  if (!encode_tmap_2d(&map_a, a_mat, uint64_t(P) * m_shard, k, 2, gemm::BM) ||
      !encode_tmap_2d(&map_b, b, n, k, 2, gemm::BN / 2)) {
    return -1;
  }
  RsArgs a{team, static_cast<__nv_bfloat16 *>(staging), static_cast<__nv_bfloat16 *>(out), m_shard, n, k,
           grid_counter, epoch};
  if (use_two_cta() && m_shard % (2 * gemm2::BM) == 0 && device_sm_count() % 2 == 0) {
    cudaError_t e = cudaFuncSetAttribute(gemm_rs_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm2::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    return launch_pes(gemm_rs_pair_kernel, device_sm_count(), gemm2::THREADS, gemm2::SMEM_BYTES,
                      static_cast<cudaStream_t>(stream), true, map_a, map_b, a);
  }
  if (int rc = prepare_smem(gemm_rs_kernel)) return rc;
  return launch_pes(gemm_rs_kernel, device_sm_count(), gemm::THREADS, gemm::SMEM_BYTES,
                    static_cast<cudaStream_t>(stream), true, map_a, map_b, a);
}

int ag_gemm_fp8(rocshmem_team_t team, const void *x_q, const float *x_s, void *gathered_q, float *gathered_s,
                unsigned long long *flags, const void *b_q, const float *b_scale, void *c, int m_shard, int n, int k,
                unsigned epoch, int swiglu, void *stream) {
  Runtime &rt = Runtime::instance();
  HostTeam *ht = rt.team_from_handle(team);
  if (!ht || rt.n_local() != 1) return cudaErrorInvalidValue;
  const int P = ht->world.size;
  if (m_shard <= 0 || m_shard % gemm8::BM || n <= 0 || n % 128 || k <= 0 || k % 512) return cudaErrorInvalidValue;
  if (swiglu && (n % 256) != 0) return cudaErrorInvalidValue;
  CUtensorMap map_a, map_b;
  if (!encode_tmap_2d(&map_a, gathered_q, uint64_t(P) * m_shard, k, 1, gemm8::BM) ||
      !encode_tmap_2d(&map_b, b_q, n, k, 1, gemm8::BN / 2)) {
    return -1;
  }
  Ag8Args a{team, static_cast<const unsigned char *>(x_q), x_s, static_cast<unsigned char *>(gathered_q), gathered_s,
            reinterpret_cast<unsigned int *>(flags), b_scale, static_cast<__nv_bfloat16 *>(c), m_shard, n, k, epoch};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int sms = device_sm_count();
  auto launch = [&](auto kernel) -> int {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm8::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    return launch_pes(kernel, sms, gemm8::THREADS + 32, gemm8::SMEM_BYTES, s, true, map_a, map_b, a);
  };
  return swiglu ? launch(ag_gemm_fp8_kernel<true>) : launch(ag_gemm_fp8_kernel<false>);
}

int gemm_rs_fp8(rocshmem_team_t team, const void *a_q, const float *a_scale, const void *b_q, const float *b_scale,
                void *staging, void *out, int m_shard, int n, int k, unsigned long long *grid_counter, unsigned epoch,
                void *stream) {
  Runtime &rt = Runtime::instance();
  HostTeam *ht = rt.team_from_handle(team);
  if (!ht || rt.n_local() != 1) return cudaErrorInvalidValue;
  const int P = ht->world.size;
  if (m_shard <= 0 || m_shard % gemm8::BM || n <= 0 || n % 128 || k <= 0 || k % 512) return cudaErrorInvalidValue;
  CUtensorMap map_a, map_b;
  if (!encode_tmap_2d(&map_a, a_q, uint64_t(P) * m_shard, k, 1, gemm8::BM) ||
      !encode_tmap_2d(&map_b, b_q, n, k, 1, gemm8::BN / 2)) {
    return -1;
  }
  RsArgs a{team, static_cast<__nv_bfloat16 *>(staging), static_cast<__nv_bfloat16 *>(out), m_shard, n, k, grid_counter,
           epoch};
  auto launch = [&](auto kernel) -> int {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm8::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    return launch_pes(kernel, device_sm_count(), gemm8::THREADS, gemm8::SMEM_BYTES, static_cast<cudaStream_t>(stream),
                      true, map_a, map_b, a_scale, b_scale, a);
  };
  return launch(gemm_rs_fp8_kernel);
}

}  // namespace kernels
}  // namespace rocshmem
