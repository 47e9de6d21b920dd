// Tensor-parallel GEMMs fused with their collective, on heap-resident operands (one PE per process).
//
// all-gather -> GEMM (ag_gemm_bf16): one kernel, two kinds of CTA. A few "comm" CTAs pull the peers'
// activation shards over NVLink into a local gathered buffer with untiled bulk copies through
// shared memory (remote global -> smem -> local global, tens of KiB in flight per CTA, no threads
// busy copying), row block by row block in a rank-rotated order that starts with the local shard, and
// bump a per-row-block counter when a block is complete. All other CTAs run the tcgen05 GEMM core
// over the row blocks in the same order; the TMA producer of a CTA waits for its row block's counter
// before loading A. The transfer of later row blocks overlaps the math on earlier ones. Remote rows
// cross NVLink once (every CTA then reads them from local HBM / L2).
//
// GEMM -> reduce-scatter (gemm_rs_bf16): the GEMM epilogue stores each finished 128 x 256 tile
// straight into the staging buffer of the rank that owns those rows (16-byte peer stores), tiles
// ordered so that the ranks write to different owners at any time and a rank's own rows come last.
// After a cross-rank barrier every CTA sums its share of the n_ranks staged partials of the local
// rows in fp32 and writes the bf16 result.
//
// Nothing here has a counterpart in the reference; the ingredients it offers are fcollect, reduction
// and put-with-signal (src/ipc/context_ipc_tmpl_device.hpp:166-531).
#include <cuda.h>
#include <cuda_bf16.h>

#include "gemm_core.cuh"
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

constexpr int kPieceBytes = 32 * 1024;
constexpr int kCopyBuffers = 5;  // 160 KiB of loads in flight per comm CTA

struct AgArgs {
  rocshmem_team_t team;
  const __nv_bfloat16 *x_shard;   // symmetric [m_shard, k]
  __nv_bfloat16 *gathered;        // local [n_ranks * m_shard, k]
  unsigned int *ready;            // local [n_ranks * m_shard / 128], monotonic
  __nv_bfloat16 *c;
  int m_shard, n, k;
  unsigned epoch;
  int comm_blocks;
};

// With SWIGLU the weight holds gate rows [0, n / 2) and up rows [n / 2, n); one tile pairs 128 gate
// columns with the matching up columns and the output is silu(gate) * up of width n / 2.
template <bool SWIGLU>
struct AgScheduler {
  int me, n_ranks, tiles_per_shard, tiles_n, tiles, m_shard, n, comm_blocks;
  const unsigned int *ready_count;
  unsigned target;
  __device__ bool get(int iter, gemm::Tile &t) const {
    const int id = (blockIdx.x - comm_blocks) + iter * (gridDim.x - comm_blocks);
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
  __device__ bool ready_wait(const unsigned int *p) const {
    if (*reinterpret_cast<const volatile unsigned int *>(p) >= target) return true;
    detail::SpinBudget budget(gemm::WAIT_BUDGET_NS);
    while (*reinterpret_cast<const volatile unsigned int *>(p) < target) {
      if (!budget.keep_going()) return false;
    }
    return true;
  }
  __device__ bool ready(const gemm::Tile &t) const {
    if (!ready_wait(ready_count + t.tag)) return false;
    __threadfence();
    sm100::fence_proxy_async();  // the rows were written through the async proxy and are read by TMA
    return true;
  }
};

struct PlainEpilogue {
  __nv_bfloat16 *c;
  size_t ldc;
  __device__ __nv_bfloat16 *row_ptr(const gemm::Tile &t, int row) const {
    return c + static_cast<size_t>(t.c_row + row) * ldc + t.c_col;
  }
};

// What the comm CTAs move: row blocks of 128 rows from every member's symmetric `src` into the local
// `dst` (block b of member s lands at block s * tiles_per_shard + b), optionally together with a second,
// smaller array (`src2` -> `dst2`: the rows' fp8 scales) that every comm CTA moves an equal slice of.
struct AgComm {
  const char *src;    // symmetric, tiles_per_shard * tile_bytes
  char *dst;          // local, n_ranks * tiles_per_shard * tile_bytes
  size_t tile_bytes;  // multiple of 16
  const char *src2;
  char *dst2;
  size_t tile2_bytes; // 0: none; else a multiple of 16 * comm_blocks
  int tiles_per_shard;
  unsigned int *ready;  // local [n_ranks * tiles_per_shard], monotonic: += comm_blocks per call
  int comm_blocks;
};

// One thread of a comm CTA moves this CTA's share of every row block: pieces c, c + C, c + 2C, ... of
// the first array and slice c of the second.
__device__ void ag_comm_role(const AgComm &a, const rocshmem_team_dev *t, unsigned char *smem_raw) {
  __shared__ uint64_t s_full[kCopyBuffers];
  __shared__ int s_abort;
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int C = a.comm_blocks, c = blockIdx.x;
  const int P = t->size, me = t->my_pe;
  if (threadIdx.x == 0) {
    for (int b = 0; b < kCopyBuffers; ++b) sm100::mbar_init(&s_full[b], 1);
    s_abort = 0;
    sm100::mbar_fence_init();
  }
  // Every member's shard is complete (its producers ran before this kernel on its stream).
  bool ok = block_pair_barrier(t, blockIdx.x);
  if (ok && threadIdx.x == 0) {
    const int ppt = static_cast<int>((a.tile_bytes + kPieceBytes - 1) / kPieceBytes);  // pieces per row block
    const int data_per_tile = (ppt - c + C - 1) / C;                  // pieces of a row block that are mine
    const int per_tile = data_per_tile + (a.tile2_bytes ? 1 : 0);
    const size_t slice2 = a.tile2_bytes / C;
    const long total = long(P) * a.tiles_per_shard * per_tile;
    // Piece j: source address, destination address and length.
    auto piece = [&](long j, const char *&src, char *&dst, uint32_t &len) {
      const long tile = j / per_tile;
      const int sub = int(j % per_tile);
      const int s = (me + int(tile / a.tiles_per_shard)) % P, mt = int(tile % a.tiles_per_shard);
      const int world_pe = team_pe_to_world(t, s);
      const size_t dst_tile = size_t(s) * a.tiles_per_shard + mt;
      if (sub < data_per_tile) {
        const size_t off = size_t(c + sub * C) * kPieceBytes;
        src = remote_ptr(a.src, world_pe) + size_t(mt) * a.tile_bytes + off;
        dst = a.dst + dst_tile * a.tile_bytes + off;
        const size_t left = a.tile_bytes - off;
        len = static_cast<uint32_t>(left < size_t(kPieceBytes) ? left : size_t(kPieceBytes));
      } else {
        const size_t off = size_t(c) * slice2;
        src = remote_ptr(a.src2, world_pe) + size_t(mt) * a.tile2_bytes + off;
        dst = a.dst2 + dst_tile * a.tile2_bytes + off;
        len = static_cast<uint32_t>(slice2);
      }
    };
    const long prefill = total < kCopyBuffers ? total : kCopyBuffers;
    for (long j = 0; j < prefill; ++j) {
      const char *src; char *dst; uint32_t len;
      piece(j, src, dst, len);
      sm100::mbar_arrive_expect_tx(&s_full[j], len);
      sm100::bulk_load(smem + j * kPieceBytes, src, len, &s_full[j]);
    }
    for (long j = 0; j < total; ++j) {
      const int b = int(j % kCopyBuffers);
      const uint32_t parity = uint32_t(j / kCopyBuffers) & 1u;
      const char *src; char *dst; uint32_t len;
      piece(j, src, dst, len);
      if (!sm100::mbar_wait(&s_full[b], parity, &s_abort, gemm::WAIT_BUDGET_NS)) {
        detail::record_error(ROCSHMEM_ERR_KERNEL, -1, 80, src, j, 0);
        break;
      }
      sm100::bulk_store(dst, smem + b * kPieceBytes, len);
      sm100::bulk_commit();
      const bool tile_done = ((j + 1) % per_tile) == 0;
      if (tile_done) {
        // All stores of this row block have completed (not only been read from shared memory).
        sm100::bulk_wait_all();
        sm100::fence_proxy_async();
        __threadfence();
        atomicAdd(a.ready + j / per_tile, 1u);
      } else {
        sm100::bulk_wait_read_all();  // the buffer may be refilled once the store has read it
      }
      if (j + kCopyBuffers < total) {
        const char *nsrc; char *ndst; uint32_t nlen;
        piece(j + kCopyBuffers, nsrc, ndst, nlen);
        sm100::mbar_arrive_expect_tx(&s_full[b], nlen);
        sm100::bulk_load(smem + b * kPieceBytes, nsrc, nlen, &s_full[b]);
      }
    }
    sm100::bulk_wait_all();
  }
  // Peers may overwrite their shards once everybody has finished pulling.
  block_pair_barrier(t, blockIdx.x, false);
}

template <bool SWIGLU>
__global__ void __launch_bounds__(gemm::THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, AgArgs a) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm::Shared sh;
  const rocshmem_team_dev *t = detail::team_of(a.team);
  if (t->my_pe < 0) return;
  if (static_cast<int>(blockIdx.x) < a.comm_blocks) {
    const AgComm comm{reinterpret_cast<const char *>(a.x_shard), reinterpret_cast<char *>(a.gathered),
                      size_t(gemm::BM) * a.k * 2, nullptr, nullptr, 0, a.m_shard / gemm::BM, a.ready, a.comm_blocks};
    ag_comm_role(comm, t, smem_raw);
    return;
  }
  AgScheduler<SWIGLU> sched;
  sched.me = t->my_pe;
  sched.n_ranks = t->size;
  sched.tiles_per_shard = a.m_shard / gemm::BM;
  sched.tiles_n = SWIGLU ? (a.n / 2 + gemm::BN / 2 - 1) / (gemm::BN / 2) : (a.n + gemm::BN - 1) / gemm::BN;
  sched.tiles = t->size * sched.tiles_per_shard * sched.tiles_n;
  sched.m_shard = a.m_shard;
  sched.n = a.n;
  sched.comm_blocks = a.comm_blocks;
  sched.ready_count = a.ready;
  sched.target = a.epoch * static_cast<unsigned>(a.comm_blocks);
  PlainEpilogue epi{a.c, static_cast<size_t>(SWIGLU ? a.n / 2 : a.n)};
  gemm::run<false, SWIGLU>(&map_a, &map_b, a.k * 2, sched, epi, smem_raw, sh);
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
};

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

// ---- block-scaled e4m3 variants -------------------------------------------------------------------------------
// Same structure with the fp8 core: the comm CTAs gather the e4m3 rows and, as a second array, their
// 1 x 128 scales (half the NVLink bytes of the bf16 kernel); the weights carry 128 x 128 scales.

struct Ag8Args {
  rocshmem_team_t team;
  const unsigned char *x_q;   // symmetric [m_shard, k] e4m3
  const float *x_s;           // symmetric [m_shard, k / 128]
  unsigned char *gathered_q;  // local [n_ranks * m_shard, k]
  float *gathered_s;          // local [n_ranks * m_shard, k / 128]
  unsigned int *ready;
  const float *b_scale;
  __nv_bfloat16 *c;
  int m_shard, n, k;
  unsigned epoch;
  int comm_blocks;
};

template <bool SWIGLU>
__global__ void __launch_bounds__(gemm8::THREADS, 1)
ag_gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, Ag8Args a) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ gemm8::Shared sh;
  const rocshmem_team_dev *t = detail::team_of(a.team);
  if (t->my_pe < 0) return;
  if (static_cast<int>(blockIdx.x) < a.comm_blocks) {
    const AgComm comm{reinterpret_cast<const char *>(a.x_q), reinterpret_cast<char *>(a.gathered_q),
                      size_t(gemm8::BM) * a.k, reinterpret_cast<const char *>(a.x_s),
                      reinterpret_cast<char *>(a.gathered_s), size_t(gemm8::BM) * (a.k / 128) * sizeof(float),
                      a.m_shard / gemm8::BM, a.ready, a.comm_blocks};
    ag_comm_role(comm, t, smem_raw);
    return;
  }
  AgScheduler<SWIGLU> sched;
  sched.me = t->my_pe;
  sched.n_ranks = t->size;
  sched.tiles_per_shard = a.m_shard / gemm8::BM;
  sched.tiles_n = SWIGLU ? (a.n / 2 + gemm8::BN / 2 - 1) / (gemm8::BN / 2) : (a.n + gemm8::BN - 1) / gemm8::BN;
  sched.tiles = t->size * sched.tiles_per_shard * sched.tiles_n;
  sched.m_shard = a.m_shard;
  sched.n = a.n;
  sched.comm_blocks = a.comm_blocks;
  sched.ready_count = a.ready;
  sched.target = a.epoch * static_cast<unsigned>(a.comm_blocks);
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
  gemm8::run<false>(&map_a, &map_b, a_scale, b_scale, a.k / gemm8::KB, sched, epi, smem_raw, sh);
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
                 const void *b, void *c, int m_shard, int n, int k, unsigned epoch, int comm_blocks,
                 int swiglu, void *stream) {
  Runtime &rt = Runtime::instance();
  HostTeam *ht = rt.team_from_handle(team);
  if (!ht || rt.n_local() != 1) return cudaErrorInvalidValue;
  const int P = ht->world.size;
  if (m_shard <= 0 || m_shard % gemm::BM || n <= 0 || n % 8 || k <= 0 || k % 128) return cudaErrorInvalidValue;
  const int ppt = static_cast<int>(size_t(gemm::BM) * k * 2 / kPieceBytes);
  if (ppt < 1) return cudaErrorInvalidValue;
  const int sms = device_sm_count();
  comm_blocks = std::max(1, std::min(std::min(comm_blocks, ppt), sms / 4));
  CUtensorMap map_a, map_b;
  if (!encode_tmap_2d(&map_a, gathered, uint64_t(P) * m_shard, k, 2, gemm::BM) ||
      !encode_tmap_2d(&map_b, b, n, k, 2, gemm::BN / 2)) {
    return -1;
  }
  if (swiglu && (n % 16) != 0) return cudaErrorInvalidValue;
  if (int rc = swiglu ? prepare_smem(ag_gemm_kernel<true>) : prepare_smem(ag_gemm_kernel<false>)) return rc;
  AgArgs a{team, static_cast<const __nv_bfloat16 *>(x_shard), static_cast<__nv_bfloat16 *>(gathered),
           reinterpret_cast<unsigned int *>(flags), static_cast<__nv_bfloat16 *>(c), m_shard, n, k, epoch,
           comm_blocks};
  // Comm CTAs wait for peers, GEMM CTAs wait for comm CTAs: all of them must be resident.
  if (swiglu) {
    return launch_pes(ag_gemm_kernel<true>, sms, gemm::THREADS, gemm::SMEM_BYTES, static_cast<cudaStream_t>(stream),
                      true, map_a, map_b, a);
  }
  return launch_pes(ag_gemm_kernel<false>, sms, gemm::THREADS, gemm::SMEM_BYTES, static_cast<cudaStream_t>(stream),
                    true, map_a, map_b, a);
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
  if (int rc = prepare_smem(gemm_rs_kernel)) return rc;
  RsArgs a{team, static_cast<__nv_bfloat16 *>(staging), static_cast<__nv_bfloat16 *>(out), m_shard, n, k,
           grid_counter, epoch};
  return launch_pes(gemm_rs_kernel, device_sm_count(), gemm::THREADS, gemm::SMEM_BYTES,
                    static_cast<cudaStream_t>(stream), true, map_a, map_b, a);
}

int ag_gemm_fp8(rocshmem_team_t team, const void *x_q, const float *x_s, void *gathered_q, float *gathered_s,
                unsigned long long *flags, const void *b_q, const float *b_scale, void *c, int m_shard, int n, int k,
                unsigned epoch, int comm_blocks, int swiglu, void *stream) {
  Runtime &rt = Runtime::instance();
  HostTeam *ht = rt.team_from_handle(team);
  if (!ht || rt.n_local() != 1) return cudaErrorInvalidValue;
  const int P = ht->world.size;
  if (m_shard <= 0 || m_shard % gemm8::BM || n <= 0 || n % 128 || k <= 0 || k % 512) return cudaErrorInvalidValue;
  if (swiglu && (n % 256) != 0) return cudaErrorInvalidValue;
  const int ppt = static_cast<int>((size_t(gemm8::BM) * k + kPieceBytes - 1) / kPieceBytes);
  const int sms = device_sm_count();
  comm_blocks = std::max(1, std::min(std::min(comm_blocks, ppt), sms / 4));
  // Every comm CTA moves an equal, 16-byte aligned slice of a row block's scales (128 * k / 128 floats).
  const size_t tile2 = size_t(gemm8::BM) * (k / 128) * sizeof(float);
  while (comm_blocks > 1 && (tile2 % (size_t(16) * comm_blocks)) != 0) --comm_blocks;
  CUtensorMap map_a, map_b;
  if (!encode_tmap_2d(&map_a, gathered_q, uint64_t(P) * m_shard, k, 1, gemm8::BM) ||
      !encode_tmap_2d(&map_b, b_q, n, k, 1, gemm8::BN / 2)) {
    return -1;
  }
  Ag8Args a{team, static_cast<const unsigned char *>(x_q), x_s, static_cast<unsigned char *>(gathered_q), gathered_s,
            reinterpret_cast<unsigned int *>(flags), b_scale, static_cast<__nv_bfloat16 *>(c), m_shard, n, k, epoch,
            comm_blocks};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (swiglu) {
    cudaError_t e = cudaFuncSetAttribute(ag_gemm_fp8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm8::SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    return launch_pes(ag_gemm_fp8_kernel<true>, sms, gemm8::THREADS, gemm8::SMEM_BYTES, s, true, map_a, map_b, a);
  }
  cudaError_t e = cudaFuncSetAttribute(ag_gemm_fp8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm8::SMEM_BYTES);
  if (e != cudaSuccess) return static_cast<int>(e);
  return launch_pes(ag_gemm_fp8_kernel<false>, sms, gemm8::THREADS, gemm8::SMEM_BYTES, s, true, map_a, map_b, a);
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
  cudaError_t e = cudaFuncSetAttribute(gemm_rs_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm8::SMEM_BYTES);
  if (e != cudaSuccess) return static_cast<int>(e);
  RsArgs a{team, static_cast<__nv_bfloat16 *>(staging), static_cast<__nv_bfloat16 *>(out), m_shard, n, k, grid_counter,
           epoch};
  return launch_pes(gemm_rs_fp8_kernel, device_sm_count(), gemm8::THREADS, gemm8::SMEM_BYTES,
                    static_cast<cudaStream_t>(stream), true, map_a, map_b, a_scale, b_scale, a);
}

}  // namespace kernels
}  // namespace rocshmem
