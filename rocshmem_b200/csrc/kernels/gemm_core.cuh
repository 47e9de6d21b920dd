// Persistent, warp-specialised tcgen05 GEMM core shared by the plain, grouped and fused kernels.
//
// One CTA per SM computes 128 x 256 output tiles of C = A * B^T (A [*, K] and B [*, K] both K-major):
//   warp 0      TMA producer: per 128-byte K slab one 128-row box of A and two 128-row boxes of B land
//               in a 4-stage shared-memory ring (128-byte swizzle), completion on mbarriers;
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M 128, N 256, K 32 bytes per
//               instruction) into one of two 256-column TMEM accumulators and commits to mbarriers that
//               free the smem stage / publish the finished accumulator;
//   warps 2..5  epilogue: tcgen05.ld of 32-column chunks, conversion, stores. While they drain one
//               accumulator the MMA warp already fills the other one.
// Policies supply the tile order (Scheduler), a hook the producer calls before it loads a tile's A
// rows (used to wait for rows that another GPU is still sending) and the epilogue's destination.
// A rows can also be gathered by index (warps 6..9 instead of TMA: cp.async copies of each row's 128 bytes of the K
// slab into the stage with the 128-byte swizzle, eight lanes per row), and the epilogue can scale rows and add
// them into the destination instead of storing them.
// Every wait is bounded; on expiry the CTA sets its abort flag, all roles leave their loops, TMEM is
// freed and a global error counter is bumped.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <type_traits>

#include "sm100_ptx.cuh"

namespace rocshmem {
namespace kernels {
namespace gemm {

constexpr int BM = 128;            // rows of A per tile (UMMA M)
constexpr int BN = 256;            // rows of B per tile (UMMA N)
constexpr int SLAB_BYTES = 128;    // K extent of one stage in bytes (one swizzle atom)
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * SLAB_BYTES;        // 16 KiB
constexpr int B_STAGE_BYTES = BN * SLAB_BYTES;        // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int EPI_COLS = 64;                            // output columns staged per step
constexpr int EPI_ROW_BYTES = EPI_COLS * 2 + 16;        // padded: conflict-free 16-byte accesses
constexpr int EPI_WARP_BYTES = 32 * EPI_ROW_BYTES;      // one staging area per epilogue warp
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 4 * EPI_WARP_BYTES + 1024;  // + slack for 1024-byte alignment
constexpr int THREADS = 192;
constexpr int GATHER_WARPS = 4;                    // extra warps of kernels whose A rows are gathered by index
constexpr int GATHER_THREADS = THREADS + GATHER_WARPS * 32;
constexpr int TMEM_COLS = 512;     // two accumulators of 256 fp32 columns
constexpr unsigned long long WAIT_BUDGET_NS = 2000000000ull;  // 2 s per wait

struct Tile {
  int a_row;      // first row of the A box (tensor-map coordinate)
  int b_row[2];   // first rows of the two 128-row B boxes
  int rows;       // valid rows in this tile (<= 128); rows beyond are computed but not stored
  int cols;       // valid output columns (<= 256, or <= 128 with SwiGLU)
  int c_row;      // output row of tile row 0
  int c_col;      // output column of tile column 0
  int tag;        // scheduler-defined (e.g. index of the row block in arrival order)
};

// Maps a linear tile id to (row block, column tile). Row blocks are taken in groups of `group` and a
// group is swept column by column: CTAs that run at the same time share `group` row blocks of A
// (which stay in L2) and a handful of B tiles, and B is streamed from HBM once per group instead of
// once per row block. Matters as soon as B is larger than L2.
constexpr int RASTER_GROUP = 8;
__device__ __forceinline__ void raster(int id, int row_blocks, int tiles_n, int group, int &rb, int &nt) {
  const int per_group = group * tiles_n;
  const int g = id / per_group, rem = id - g * per_group;
  const int rows = min(group, row_blocks - g * group);
  nt = rem / rows;
  rb = g * group + rem % rows;
}

// One counter per translation unit (the kernels are not built as relocatable device code).
static __device__ unsigned int g_gemm_errors = 0;

// Where the A rows come from when they are gathered: tile row r of a tile reads source row
// row_index[t.a_row + r], which holds the MMA's element type (row_bytes = K * element size). The block-scaled core
// also reads the rows' scales through the index (`scales` [rows, nscale]).
struct GatherSrc {
  const int *row_index;
  const unsigned char *base;
  size_t row_bytes;
  const float *scales;
  int nscale;
};

// Write-out of one warp's staged 32 x 64 bf16 block (padded rows in shared memory), 8 lanes per row, shared by the
// one-CTA and the two-CTA cores.
template <bool EPI_ADD, class Epilogue>
__device__ __forceinline__ void write_out_block(const Tile &t, Epilogue &epi, const unsigned char *stg, int row0,
                                                int col0, int lane) {
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 4 + lane / 8, seg = lane % 8;
    const int row = row0 + r, col = col0 + seg * 8;
    if (row >= t.rows || col >= t.cols) continue;
    __nv_bfloat16 *out = epi.row_ptr(t, row);
    if (out == nullptr) continue;
    const unsigned char *src = stg + r * EPI_ROW_BYTES + seg * 16;
    __nv_bfloat16 *dst = out + col;
    if (col + 8 <= t.cols && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
      const int4 val = *reinterpret_cast<const int4 *>(src);
      if (EPI_ADD) sm100::red_add_bf16x8(dst, val);
      else *reinterpret_cast<int4 *>(dst) = val;
    } else {
      const __nv_bfloat16 *s16 = reinterpret_cast<const __nv_bfloat16 *>(src);
      for (int i = 0; i < 8 && col + i < t.cols; ++i) {
        if (EPI_ADD) atomicAdd(dst + i, s16[i]);
        else dst[i] = s16[i];
      }
    }
  }
}

struct Shared {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

// Scheduler: struct with  __device__ bool get(int iter, Tile &t)  (false: no more tiles for this CTA),
//                         __device__ bool ready(const Tile &t)    (producer-side hook, bounded; false aborts)
//            and          __device__ void side_role()             (run by warps beyond the six of the GEMM,
//                                                                  if the kernel is launched with any).
// Epilogue:  struct with  __device__ __nv_bfloat16 *row_ptr(const Tile &t, int row_in_tile)
//            returning the address of output element (row, t.c_col), or nullptr to skip the row; with EPI_ADD
//            also  __device__ float row_scale(const Tile &t, int row_in_tile)  and the rows are multiplied by it
//            and added to the destination (red.global.add on packed bf16) instead of stored.
template <bool IS_FP8, bool SWIGLU, bool A_GATHER = false, bool EPI_ADD = false, class Scheduler, class Epilogue>
__device__ __forceinline__ void run(const CUtensorMap *map_a, const CUtensorMap *map_b, int k_bytes,
                                    Scheduler &sched, Epilogue &epi, unsigned char *smem_raw, Shared &sh,
                                    const GatherSrc *gather = nullptr) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int k_slabs = (k_bytes + SLAB_BYTES - 1) / SLAB_BYTES;
  constexpr int ELEM_BYTES = IS_FP8 ? 1 : 2;
  constexpr int SLAB_ELEMS = SLAB_BYTES / ELEM_BYTES;
  constexpr uint32_t IDESC = sm100::make_idesc(BM, BN, IS_FP8 ? sm100::kFormatE4M3 : sm100::kFormatBF16);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      // Gathered A: the stage is full when the B bytes have landed and every gather thread has stored its row.
      sm100::mbar_init(&sh.full[s], A_GATHER ? 1 + GATHER_WARPS * 32 : 1);
      sm100::mbar_init(&sh.empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      sm100::mbar_init(&sh.tmem_full[a], 1);
      sm100::mbar_init(&sh.tmem_empty[a], 4);
    }
    sh.abort_flag = 0;
    sm100::mbar_fence_init();
    if (!A_GATHER) sm100::tma_prefetch_desc(map_a);
    sm100::tma_prefetch_desc(map_b);
  }
  if (warp == 1) sm100::tmem_alloc(&sh.tmem_base, TMEM_COLS);
  sm100::tcgen05_fence_before();
  __syncthreads();
  sm100::tcgen05_fence_after();
  const uint32_t tmem_base = sh.tmem_base;

  if (warp == 0) {
    // ---- producer ---------------------------------------------------------------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      Tile t;
      for (int iter = 0; sched.get(iter, t) && !sh.abort_flag; ++iter) {
        if (!sched.ready(t)) {
          sh.abort_flag = 1;
          break;
        }
        for (int ks = 0; ks < k_slabs; ++ks) {
          if (!sm100::mbar_wait(&sh.empty[stage], phase ^ 1u, &sh.abort_flag, WAIT_BUDGET_NS)) break;
          unsigned char *sa = smem + stage * STAGE_BYTES;
          unsigned char *sb = sa + A_STAGE_BYTES;
          sm100::mbar_arrive_expect_tx(&sh.full[stage], A_GATHER ? B_STAGE_BYTES : STAGE_BYTES);
          if (!A_GATHER) sm100::tma_load_2d(sa, map_a, &sh.full[stage], ks * SLAB_ELEMS, t.a_row);
          sm100::tma_load_2d(sb, map_b, &sh.full[stage], ks * SLAB_ELEMS, t.b_row[0]);
          sm100::tma_load_2d(sb + B_STAGE_BYTES / 2, map_b, &sh.full[stage], ks * SLAB_ELEMS, t.b_row[1]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (sh.abort_flag) break;
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer --------------------------------------------------------------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      Tile t;
      for (int iter = 0; sched.get(iter, t) && !sh.abort_flag; ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1u;
        if (!sm100::mbar_wait(&sh.tmem_empty[acc], acc_phase ^ 1u, &sh.abort_flag, WAIT_BUDGET_NS)) break;
        sm100::tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int ks = 0; ks < k_slabs; ++ks) {
          if (!sm100::mbar_wait(&sh.full[stage], phase, &sh.abort_flag, WAIT_BUDGET_NS)) break;
          sm100::tcgen05_fence_after();
          // Gathered rows were written through the generic proxy (cp.async, st.shared); the MMA reads them through
          // the async proxy.
          if (A_GATHER) sm100::fence_proxy_async_smem();
          const uint32_t sa = sm100::smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
          const uint64_t da = sm100::make_sw128_desc(sa), db = sm100::make_sw128_desc(sb);
#pragma unroll
          for (int kk = 0; kk < SLAB_BYTES / 32; ++kk) {
            // Each instruction consumes 32 bytes of K; advancing the start address by 32 bytes (2 in
            // 16-byte units) inside the swizzle atom selects the next K chunk.
            if (IS_FP8) sm100::mma_f8(tmem_d, da + 2 * kk, db + 2 * kk, IDESC, (ks | kk) != 0);
            else sm100::mma_f16(tmem_d, da + 2 * kk, db + 2 * kk, IDESC, (ks | kk) != 0);
          }
          sm100::mma_commit(&sh.empty[stage]);  // frees the smem stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (sh.abort_flag) break;
        sm100::mma_commit(&sh.tmem_full[acc]);  // accumulator complete
      }
    }
  } else if (A_GATHER && warp >= 6 && warp < 6 + GATHER_WARPS) {
    // ---- gather producers -----------------------------------------------------------------------------------------
    // Lanes are laid out so that neighbouring lanes read neighbouring 16-byte pieces of one row (a warp instruction
    // then touches 4 or 8 lines, not 32): warp w serves tile rows [32 w, 32 w + 32).
    const int gw = warp - 6;
    uint32_t stage = 0, phase = 0;
    Tile t;
    for (int iter = 0; sched.get(iter, t) && !sh.abort_flag; ++iter) {
      bool ok = true;
      {
        // Rows have the MMA's element type: asynchronous 16-byte copies straight into the stage, eight
        // lanes per row (128 contiguous bytes), four rows per instruction, eight instructions per stage and warp.
        // The thread never waits for data, so it runs as far ahead as the ring has free stages; the stage's barrier
        // gets this thread's arrival when its copies have landed. (The MMA thread crosses to the async proxy after
        // its wait.)
        const uint32_t c = static_cast<uint32_t>(lane & 7);
        const unsigned char *src[8];
        uint32_t dst_off[8];
        uint32_t live_bytes[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int r = gw * 32 + j * 4 + lane / 8;
          const bool live = r < t.rows;
          const long long src_row = live ? gather->row_index[t.a_row + r] : 0;
          src[j] = gather->base + static_cast<size_t>(src_row) * gather->row_bytes + c * 16;
          dst_off[j] = static_cast<uint32_t>(r) * SLAB_BYTES + ((c ^ static_cast<uint32_t>(r & 7)) << 4);
          live_bytes[j] = live ? 16u : 0u;
        }
        for (int ks = 0; ks < k_slabs; ++ks) {
          if (!sm100::mbar_wait(&sh.empty[stage], phase ^ 1u, &sh.abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
          unsigned char *sa = smem + stage * STAGE_BYTES;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            sm100::cp_async_16(sa + dst_off[j], src[j] + static_cast<size_t>(ks) * SLAB_BYTES, live_bytes[j]);
          }
          sm100::cp_async_arrive_noinc(&sh.full[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok || sh.abort_flag) break;
    }
  } else if (warp >= 6) {
    // ---- optional extra warps (kernels launched with more than THREADS threads) ------------------------------
    sched.side_role();
  } else {
    // ---- epilogue -------------------------------------------------------------------------------------------
    // A thread receives one accumulator row from TMEM. Stores of one row per thread would scatter 16-byte
    // pieces over 32 rows per instruction (costly for local memory, ruinous over NVLink), so every warp
    // passes 64 output columns at a time through its own padded staging rows in shared memory and writes
    // them out with 8 lanes per row: 128 contiguous bytes per row, 4 rows per instruction.
    const int quarter = warp & 3;  // TMEM lanes [32 * quarter, +32) belong to this warp
    unsigned char *stg = smem + STAGES * STAGE_BYTES + (warp - 2) * EPI_WARP_BYTES;
    Tile t;
    for (int iter = 0; sched.get(iter, t) && !sh.abort_flag; ++iter) {
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1u;
      if (!sm100::mbar_wait(&sh.tmem_full[acc], acc_phase, &sh.abort_flag, WAIT_BUDGET_NS)) break;
      sm100::tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      constexpr int OUT_CHUNKS = (SWIGLU ? BN / 2 : BN) / EPI_COLS;
      float row_scale = 1.f;
      if constexpr (EPI_ADD) row_scale = (quarter * 32 + lane) < t.rows ? epi.row_scale(t, quarter * 32 + lane) : 0.f;
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
            for (int i = 0; i < 32; ++i) f[i] = silu(__uint_as_float(v[i])) * __uint_as_float(u[i]);
          } else {
            sm100::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
          }
          if (EPI_ADD) {
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] *= row_scale;
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
        write_out_block<EPI_ADD>(t, epi, stg, quarter * 32, c * EPI_COLS, lane);
        __syncwarp();
      }
      sm100::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&sh.tmem_empty[acc]);
    }
  }
  // ---- teardown ------------------------------------------------------------------------------------------------
  if (sh.abort_flag) {
    // Give bulk copies that are still in flight time to land before the shared memory is released.
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
  if (warp == 1) {
    sm100::tcgen05_fence_after();
    sm100::tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && sh.abort_flag) atomicAdd(&g_gemm_errors, 1u);
}

}  // namespace gemm
}  // namespace kernels
}  // namespace rocshmem
