// Two-CTA (cta_group::2) variant of the bf16 tcgen05 GEMM core: a pair of CTAs on neighbouring SMs (a
// cluster of two) computes one 256 x 256 tile. Each CTA loads its 128 rows of A and only its 128 rows of
// the 256-row B tile; the tensor cores of both SMs read both halves of B through the pair's shared
// memory. Per MMA that is 32 KB of L2 -> shared-memory traffic per CTA and stage instead of 48 KB, and
// six stages fit where the one-CTA kernel has four, which is what limits that kernel (the tensor pipe
// waits for the ring).
//
// Roles per CTA: warp 0 TMA producer (both CTAs), warp 1 MMA issuer (leader CTA only: one thread issues
// tcgen05.mma.cta_group::2 for the pair), warps 2..5 epilogue (both CTAs, each drains its own 128 rows
// from its own TMEM). Barriers: the "full" barriers live in the leader and receive the bytes of both
// CTAs' loads; "empty" and "accumulator full" are signalled in both CTAs at once with a multicast
// tcgen05.commit; the leader's "accumulator empty" barrier collects the epilogue warps of both CTAs
// (the peer's arrive remotely). No TMA load uses multicast. All waits are bounded.
#pragma once

#include <cuda_bf16.h>

#include "gemm_core.cuh"
#include "sm100_ptx.cuh"

namespace rocshmem {
namespace kernels {
namespace gemm2 {

constexpr int BM = 128;            // rows of A per CTA (the pair covers 256)
constexpr int BN = 256;            // columns of the tile; each CTA loads BN / 2 rows of B
constexpr int SLAB_BYTES = 128;
constexpr int STAGES = 6;
constexpr int A_STAGE_BYTES = BM * SLAB_BYTES;          // 16 KiB
constexpr int B_STAGE_BYTES = (BN / 2) * SLAB_BYTES;    // 16 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int EPI_COLS = gemm::EPI_COLS;
constexpr int EPI_ROW_BYTES = gemm::EPI_ROW_BYTES;
constexpr int EPI_WARP_BYTES = gemm::EPI_WARP_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 4 * EPI_WARP_BYTES + 1024;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr unsigned long long WAIT_BUDGET_NS = gemm::WAIT_BUDGET_NS;

struct Shared {
  uint64_t full[STAGES];       // used in the leader: bytes of both CTAs' loads
  uint64_t empty[STAGES];      // per CTA, signalled by the leader's MMA thread in both
  uint64_t tmem_full[2];       // per CTA
  uint64_t tmem_empty[2];      // used in the leader: 8 arrivals (4 epilogue warps of each CTA)
  uint32_t tmem_base;
  volatile int abort_flag;
};

// ---- cluster / cta_group::2 PTX ------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `smem_addr` (a shared::cta address of this CTA) in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t mapa(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tiled load into this CTA's shared memory; the mbarrier (shared::cluster address) may belong to
// either CTA of the pair. No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const CUtensorMap *map, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(sm100::smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *smem_result, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sm100::smem_u32(smem_result)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
  uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
      : "memory");
}
// The mbarrier at this shared-memory offset completes in both CTAs of the pair once all MMAs issued so far
// have finished.
__device__ __forceinline__ void mma_commit_pair(uint64_t *bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(sm100::smem_u32(bar)), "h"(mask)
               : "memory");
}

// Scheduler::get(iter, tile) describes the tile of the PAIR: a_row is the first of its 256 rows of A,
// b_row[0] / b_row[1] the first rows of the two 128-row halves of B, rows counts valid rows out of 256.
template <bool SWIGLU, class Scheduler, class Epilogue>
__device__ __forceinline__ void run(const CUtensorMap *map_a, const CUtensorMap *map_b, int k_bytes, Scheduler &sched,
                                    Epilogue &epi, unsigned char *smem_raw, Shared &sh) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t rank = cluster_ctarank();   // 0: leader
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int k_slabs = (k_bytes + SLAB_BYTES - 1) / SLAB_BYTES;
  constexpr int SLAB_ELEMS = SLAB_BYTES / 2;
  constexpr uint32_t IDESC = sm100::make_idesc(2 * BM, BN, sm100::kFormatBF16);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      sm100::mbar_init(&sh.full[s], 1);
      sm100::mbar_init(&sh.empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      sm100::mbar_init(&sh.tmem_full[a], 1);
      sm100::mbar_init(&sh.tmem_empty[a], 8);
    }
    sh.abort_flag = 0;
    sm100::mbar_fence_init();
    sm100::tma_prefetch_desc(map_a);
    sm100::tma_prefetch_desc(map_b);
  }
  if (warp == 1) tmem_alloc_pair(&sh.tmem_base, TMEM_COLS);
  sm100::tcgen05_fence_before();
  __syncthreads();
  cluster_sync();   // both CTAs' barriers are initialised before anybody signals across the pair
  sm100::tcgen05_fence_after();
  const uint32_t tmem_base = sh.tmem_base;

  if (warp == 0) {
    // ---- producer (both CTAs): my 128 rows of A, my 128 rows of B; completion on the leader's barrier ----
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      gemm::Tile t;
      for (int iter = 0; sched.get(iter, t) && !sh.abort_flag; ++iter) {
        if (!sched.ready(t)) {
          sh.abort_flag = 1;
          break;
        }
        for (int ks = 0; ks < k_slabs; ++ks) {
          if (!sm100::mbar_wait(&sh.empty[stage], phase ^ 1u, &sh.abort_flag, WAIT_BUDGET_NS)) break;
          unsigned char *sa = smem + stage * STAGE_BYTES;
          unsigned char *sb = sa + A_STAGE_BYTES;
          const uint32_t full_leader = mapa(sm100::smem_u32(&sh.full[stage]), 0);
          if (rank == 0) sm100::mbar_arrive_expect_tx(&sh.full[stage], 2 * STAGE_BYTES);
          tma_load_2d_pair(sa, map_a, full_leader, ks * SLAB_ELEMS, t.a_row + int(rank) * BM);
          tma_load_2d_pair(sb, map_b, full_leader, ks * SLAB_ELEMS, t.b_row[rank]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (sh.abort_flag) break;
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer (leader only) ----------------------------------------------------------------------------
    if (rank == 0 && lane == 0) {
      uint32_t stage = 0, phase = 0;
      gemm::Tile t;
      for (int iter = 0; sched.get(iter, t) && !sh.abort_flag; ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1u;
        if (!sm100::mbar_wait(&sh.tmem_empty[acc], acc_phase ^ 1u, &sh.abort_flag, WAIT_BUDGET_NS)) break;
        sm100::tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int ks = 0; ks < k_slabs; ++ks) {
          if (!sm100::mbar_wait(&sh.full[stage], phase, &sh.abort_flag, WAIT_BUDGET_NS)) break;
          sm100::tcgen05_fence_after();
          const uint32_t sa = sm100::smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
          const uint64_t da = sm100::make_sw128_desc(sa), db = sm100::make_sw128_desc(sb);
#pragma unroll
          for (int kk = 0; kk < SLAB_BYTES / 32; ++kk) mma_f16_pair(tmem_d, da + 2 * kk, db + 2 * kk, IDESC, (ks | kk) != 0);
          mma_commit_pair(&sh.empty[stage]);   // frees the stage in both CTAs
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (sh.abort_flag) break;
        mma_commit_pair(&sh.tmem_full[acc]);   // accumulators complete in both CTAs
      }
    }
  } else if (warp >= 6) {
    sched.side_role();  // optional extra warps (kernels launched with more than THREADS threads)
  } else {
    // ---- epilogue (both CTAs): my 128 rows, staged write-out as in the one-CTA core ---------------------------
    const int quarter = warp & 3;
    unsigned char *stg = smem + STAGES * STAGE_BYTES + (warp - 2) * EPI_WARP_BYTES;
    gemm::Tile t;
    for (int iter = 0; sched.get(iter, t) && !sh.abort_flag; ++iter) {
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1u;
      if (!sm100::mbar_wait(&sh.tmem_full[acc], acc_phase, &sh.abort_flag, WAIT_BUDGET_NS)) break;
      sm100::tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      const int row_base = int(rank) * BM;   // my rows inside the pair's tile
      constexpr int OUT_CHUNKS = (SWIGLU ? BN / 2 : BN) / EPI_COLS;
#pragma unroll 1
      for (int c = 0; c < OUT_CHUNKS; ++c) {
        if (c * EPI_COLS >= t.cols) break;
#pragma unroll
        for (int h = 0; h < EPI_COLS / 32; ++h) {
          uint32_t v[32];
          float f[32];
          sm100::tmem_ld_32x32(taddr + c * EPI_COLS + h * 32, v);
          if (SWIGLU) {
            uint32_t u[32];
            sm100::tmem_ld_32x32(taddr + BN / 2 + c * EPI_COLS + h * 32, u);
            sm100::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = gemm::silu(__uint_as_float(v[i])) * __uint_as_float(u[i]);
          } else {
            sm100::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            int4 pk;
            __nv_bfloat162 *p2 = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
            for (int i = 0; i < 4; ++i) p2[i] = __floats2bfloat162_rn(f[q * 8 + 2 * i], f[q * 8 + 2 * i + 1]);
            *reinterpret_cast<int4 *>(stg + lane * EPI_ROW_BYTES + h * 64 + q * 16) = pk;
          }
        }
        __syncwarp();
        gemm::write_out_block<false>(t, epi, stg, row_base + quarter * 32, c * EPI_COLS, lane);
        __syncwarp();
      }
      sm100::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa(sm100::smem_u32(&sh.tmem_empty[acc]), 0));
    }
  }
  // ---- teardown: nobody leaves while the peer may still signal into, or read from, this CTA -------------------
  if (sh.abort_flag) {
    unsigned long long t0;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (int i = 0; i < 4096; ++i) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (now - t0 > 200000ull) break;
      __nanosleep(200);
    }
  }
  sm100::tcgen05_fence_before();
  __syncthreads();
  cluster_sync();
  if (warp == 1) {
    sm100::tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && sh.abort_flag) atomicAdd(&gemm::g_gemm_errors, 1u);
}

}  // namespace gemm2
}  // namespace kernels
}  // namespace rocshmem
