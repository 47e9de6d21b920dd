// Block-scaled fp8 (e4m3) GEMM core on tcgen05 / TMEM: C = (A * sa) (B * sb)^T with one fp32 scale per
// 1 x 128 block of A (per row and 128-element K block) and one per 128 x 128 block of B.
//
// The tensor core cannot apply per-K-block scales while it accumulates, so the accumulation is split:
//   warp 0      TMA producer, one 128-byte K block (128 e4m3) of a 128 x 256 tile per stage, 4 stages;
//   warp 1      MMA issuer: the four tcgen05.mma (kind::f8f6f4, K = 32 each) of a K block overwrite one
//               of two 256-column TMEM buffers, then commit to that buffer's mbarrier;
//   warps 2..9  accumulate: each thread owns one row and 128 columns (one B scale block) in registers;
//               per K block it reads the raw partial sums with tcgen05.ld and adds them multiplied by
//               sa[row, kb] * sb[col block, kb]. Two buffers let the tensor core run one K block ahead.
// At the end of a tile the registers are converted to bf16 and stored. The CUDA-core work per K block
// (128 FMAs per thread) takes about half as long as the tensor core needs for the block's MMAs.
// Waits are bounded as in gemm_core.cuh.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "gemm_core.cuh"
#include "sm100_ptx.cuh"

namespace rocshmem {
namespace kernels {
namespace gemm8 {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int KB = 128;            // elements (= bytes) of K per block and per stage
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * KB;
constexpr int B_STAGE_BYTES = BN * KB;
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int ACC_WARPS = 8;
constexpr int EPI_ROW_BYTES = 32 * 2 + 16;              // 32 staged bf16 columns per row, padded
constexpr int EPI_WARP_BYTES = 32 * EPI_ROW_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + ACC_WARPS * EPI_WARP_BYTES + 1024;
constexpr int THREADS = 64 + ACC_WARPS * 32;
constexpr int GATHER_WARPS = 2;                     // registers are granted per four warps: 10 or 12 warps cost the same
constexpr int GATHER_THREADS = THREADS + GATHER_WARPS * 32;
constexpr int TMEM_COLS = 512;
constexpr unsigned long long WAIT_BUDGET_NS = gemm::WAIT_BUDGET_NS;

struct Shared {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
  // QUANT_OUT: [tile parity][column half][row], (tile number + 1) << 32 | bits of the half's largest magnitude
  unsigned long long amax[2][2][BM];
};

// Scales: a_scale [rows of A][k_blocks] fp32 (row-major), b_scale [rows of B / 128][k_blocks] fp32.
// Scheduler / Epilogue as in gemm_core.cuh; the tile's a_row / b_row also index the scale arrays,
// and k_blocks must be a multiple of 4 (the scales are fetched four K blocks at a time). With SWIGLU
// the tile's b_row[0] / b_row[1] are the gate and up rows of 128 output columns and the result is
// silu(gate) * up (t.cols <= 128).
// EPI_ADD: rows are multiplied by epi.row_scale(t, row) and added to the destination (packed bf16 reductions) instead
// of stored. QUANT_OUT (with SWIGLU): the 128 output columns of a tile are one 1 x 128 block of the next GEMM's A
// operand; they are quantised to e4m3 here (the two threads that hold a row's halves exchange their maxima through
// shared memory) and written to epi.q_row_ptr(t, row) with the block's scale at epi.scale_ptr(t, row).
// A_GATHER: the A rows (and their scales) are picked by index: tile row r reads row gather->row_index[t.a_row + r]
// of gather->base / gather->scales. Two extra warps (threads THREADS .. GATHER_THREADS) copy the rows into the
// stage with the 128-byte swizzle (cp.async) instead of a TMA load; the kernel must then be launched with GATHER_THREADS.
template <bool SWIGLU, bool LATE_A = false, bool EPI_ADD = false, bool QUANT_OUT = false, bool A_GATHER = false,
          class Scheduler, class Epilogue>
__device__ __forceinline__ void run(const CUtensorMap *map_a, const CUtensorMap *map_b, const float *a_scale,
                                    const float *b_scale, int k_blocks, Scheduler &sched, Epilogue &epi,
                                    unsigned char *smem_raw, Shared &sh, const gemm::GatherSrc *gather = nullptr) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr uint32_t IDESC = sm100::make_idesc(BM, BN, sm100::kFormatE4M3);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      sm100::mbar_init(&sh.full[s], A_GATHER ? 1 + GATHER_WARPS * 32 : 1);
      sm100::mbar_init(&sh.empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      sm100::mbar_init(&sh.tmem_full[a], 1);
      sm100::mbar_init(&sh.tmem_empty[a], ACC_WARPS);
    }
    sh.abort_flag = 0;
    sm100::mbar_fence_init();
    if (!A_GATHER) sm100::tma_prefetch_desc(map_a);
    sm100::tma_prefetch_desc(map_b);
  }
  if (QUANT_OUT) {
    for (int i = threadIdx.x; i < 2 * 2 * BM; i += blockDim.x) (&sh.amax[0][0][0])[i] = 0ull;   // tag 0: no tile yet
  }
  if (warp == 1) sm100::tmem_alloc(&sh.tmem_base, TMEM_COLS);
  sm100::tcgen05_fence_before();
  __syncthreads();
  sm100::tcgen05_fence_after();
  const uint32_t tmem_base = sh.tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      gemm::Tile t;
      for (int iter = 0; sched.get(iter, t) && !sh.abort_flag; ++iter) {
        if (!sched.ready(t)) {
          sh.abort_flag = 1;
          break;
        }
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!sm100::mbar_wait(&sh.empty[stage], phase ^ 1u, &sh.abort_flag, WAIT_BUDGET_NS)) break;
          unsigned char *sa = smem + stage * STAGE_BYTES;
          unsigned char *sb = sa + A_STAGE_BYTES;
          sm100::mbar_arrive_expect_tx(&sh.full[stage], A_GATHER ? B_STAGE_BYTES : STAGE_BYTES);
          if (!A_GATHER) sm100::tma_load_2d(sa, map_a, &sh.full[stage], kb * KB, t.a_row);
          sm100::tma_load_2d(sb, map_b, &sh.full[stage], kb * KB, t.b_row[0]);
          sm100::tma_load_2d(sb + B_STAGE_BYTES / 2, map_b, &sh.full[stage], kb * KB, t.b_row[1]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (sh.abort_flag) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t buf = 0, buf_phase = 0;
      gemm::Tile t;
      for (int iter = 0; sched.get(iter, t) && !sh.abort_flag; ++iter) {
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!sm100::mbar_wait(&sh.tmem_empty[buf], buf_phase ^ 1u, &sh.abort_flag, WAIT_BUDGET_NS)) break;
          if (!sm100::mbar_wait(&sh.full[stage], phase, &sh.abort_flag, WAIT_BUDGET_NS)) break;
          sm100::tcgen05_fence_after();
          if (A_GATHER) sm100::fence_proxy_async_smem();   // rows written by cp.async, read by the async proxy
          const uint32_t tmem_d = tmem_base + buf * BN;
          const uint32_t sa = sm100::smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
          const uint64_t da = sm100::make_sw128_desc(sa), db = sm100::make_sw128_desc(sb);
#pragma unroll
          for (int kk = 0; kk < KB / 32; ++kk) sm100::mma_f8(tmem_d, da + 2 * kk, db + 2 * kk, IDESC, kk != 0);
          sm100::mma_commit(&sh.empty[stage]);
          sm100::mma_commit(&sh.tmem_full[buf]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          buf ^= 1u;
          if (buf == 0) buf_phase ^= 1u;
        }
        if (sh.abort_flag) break;
      }
    }
  } else if (A_GATHER && warp >= 2 + ACC_WARPS) {
    // ---- gather producers: asynchronous 16-byte copies straight into the stage, eight lanes per row (128 contiguous
    // bytes), four rows per instruction, sixteen instructions per stage and warp (warp w serves rows [64 w, 64 w + 64)).
    // No registers hold data, so the warps run as far ahead as the ring has free stages.
    const int gw = warp - 2 - ACC_WARPS;
    const uint32_t c = static_cast<uint32_t>(lane & 7);
    uint32_t stage = 0, phase = 0;
    gemm::Tile t;
    for (int iter = 0; sched.get(iter, t) && !sh.abort_flag; ++iter) {
      int rows[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int r = gw * 64 + j * 4 + lane / 8;
        rows[j] = r < t.rows ? gather->row_index[t.a_row + r] : -1;
      }
      bool ok = true;
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!sm100::mbar_wait(&sh.empty[stage], phase ^ 1u, &sh.abort_flag, WAIT_BUDGET_NS)) { ok = false; break; }
        unsigned char *sa = smem + stage * STAGE_BYTES;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int r = gw * 64 + j * 4 + lane / 8;
          const bool live = rows[j] >= 0;
          const unsigned char *gp = gather->base + static_cast<size_t>(live ? rows[j] : 0) * gather->row_bytes +
                                    static_cast<size_t>(kb) * KB + c * 16;
          sm100::cp_async_16(sa + r * KB + ((c ^ static_cast<uint32_t>(r & 7)) << 4), gp, live ? 16u : 0u);
        }
        sm100::cp_async_arrive_noinc(&sh.full[stage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      if (!ok || sh.abort_flag) break;
    }
  } else if (warp >= 2 + ACC_WARPS) {
    sched.side_role();  // optional extra warps (kernels launched with more than THREADS threads)
  } else {
    const int aw = warp - 2;           // 0..7
    const int quarter = warp & 3;      // TMEM lanes [32 * quarter, +32) are accessible to this warp
    const int half = aw / 4;
    // Plain: this thread owns TMEM columns [128 * half, +128), one B scale block.
    // SwiGLU: columns [0, 128) hold gate and [128, 256) the matching up projections; the thread owns
    // gate columns [64 * half, +64) in acc[0..63] and the same up columns in acc[64..127], so that
    // silu(gate) * up needs no exchange between threads. Gate and up have their own B scale blocks.
    const int row = quarter * 32 + lane;
    uint32_t buf = 0, buf_phase = 0;
    gemm::Tile t;
    for (int iter = 0; sched.get(iter, t) && !sh.abort_flag; ++iter) {
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.f;
      const bool row_ok = row < t.rows;
      // Gathered A: the row's scales sit with its source row.
      const size_t a_scale_row = A_GATHER ? static_cast<size_t>(gather->row_index[t.a_row + (row_ok ? row : 0)])
                                          : static_cast<size_t>(t.a_row + (row_ok ? row : 0));
      const float4 *sa4 = reinterpret_cast<const float4 *>((A_GATHER ? gather->scales : a_scale) + a_scale_row * k_blocks);
      const float4 *sb4 = reinterpret_cast<const float4 *>(b_scale + static_cast<size_t>(t.b_row[SWIGLU ? 0 : half] / 128) * k_blocks);
      const float4 *su4 = reinterpret_cast<const float4 *>(b_scale + static_cast<size_t>(t.b_row[1] / 128) * k_blocks);
      // LATE_A: the A scales of a tile may still be on their way from another GPU until the producer has
      // seen the tile's rows arrive; the first finished K block proves it has. Read past L1 (__ldcg).
      if (LATE_A && !sm100::mbar_wait(&sh.tmem_full[buf], buf_phase, &sh.abort_flag, WAIT_BUDGET_NS)) break;
      float4 a_next = __ldcg(sa4), b_next = sb4[0], u_next = make_float4(0.f, 0.f, 0.f, 0.f);
      if (SWIGLU) u_next = su4[0];
      for (int kb4 = 0; kb4 < k_blocks / 4 && !sh.abort_flag; ++kb4) {
        const float4 a_cur = a_next, b_cur = b_next, u_cur = u_next;
        if (kb4 + 1 < k_blocks / 4) {  // fetched one group ahead of its use
          a_next = __ldcg(sa4 + kb4 + 1);
          b_next = sb4[kb4 + 1];
          if (SWIGLU) u_next = su4[kb4 + 1];
        }
        const float scale[4] = {a_cur.x * b_cur.x, a_cur.y * b_cur.y, a_cur.z * b_cur.z, a_cur.w * b_cur.w};
        const float scale_u[4] = {a_cur.x * u_cur.x, a_cur.y * u_cur.y, a_cur.z * u_cur.z, a_cur.w * u_cur.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (!sm100::mbar_wait(&sh.tmem_full[buf], buf_phase, &sh.abort_flag, WAIT_BUDGET_NS)) break;
          sm100::tcgen05_fence_after();
          const uint32_t tbuf = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint32_t v[16];
            // SwiGLU: chunks 0..3 come from the gate columns, 4..7 from the up columns.
            const uint32_t col = SWIGLU ? (c < 4 ? half * 64 + c * 16 : 128 + half * 64 + (c - 4) * 16) : half * 128 + c * 16;
            const float s = (SWIGLU && c >= 4) ? scale_u[j] : scale[j];
            sm100::tmem_ld_32x16(tbuf + col, v);
            sm100::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[c * 16 + i] = fmaf(s, __uint_as_float(v[i]), acc[c * 16 + i]);
          }
          sm100::tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) sm100::mbar_arrive(&sh.tmem_empty[buf]);
          buf ^= 1u;
          if (buf == 0) buf_phase ^= 1u;
        }
      }
      if (sh.abort_flag) break;
      constexpr int OUT = SWIGLU ? 64 : 128;   // output columns per thread
      if (SWIGLU) {
#pragma unroll
        for (int i = 0; i < 64; ++i) acc[i] = gemm::silu(acc[i]) * acc[64 + i];
      }
      if constexpr (EPI_ADD) {
        const float rs = row_ok ? epi.row_scale(t, row) : 0.f;
#pragma unroll
        for (int i = 0; i < OUT; ++i) acc[i] *= rs;
      }
      const int col0 = half * OUT;
      unsigned char *stg = smem + STAGES * STAGE_BYTES + aw * EPI_WARP_BYTES;
      if constexpr (QUANT_OUT) {
        static_assert(!QUANT_OUT || SWIGLU, "the quantising epilogue belongs to the SwiGLU tile");
        // This thread holds 64 of the row's 128 columns; its partner (same row, other half) sits in another warp.
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 64; ++i) amax = fmaxf(amax, fabsf(acc[i]));
        // Value and "this is tile `iter`" travel in one 8-byte shared-memory store; the partner polls for the tag
        // (bounded, and released by the abort flag: no block-wide barrier that a role that gave up could miss).
        // Two slots alternate: a thread can only be at tile i + 2 once its partner has written tile i + 1, i.e.
        // after the partner has read tile i.
        const int par = iter & 1;
        const unsigned long long tag = static_cast<unsigned long long>(iter + 1) << 32;
        *reinterpret_cast<volatile unsigned long long *>(&sh.amax[par][half][row]) = tag | __float_as_uint(amax);
        volatile unsigned long long *theirs = &sh.amax[par][half ^ 1][row];
        unsigned long long seen = *theirs;
        for (unsigned spins = 0; (seen >> 32) != static_cast<unsigned long long>(iter + 1); seen = *theirs) {
          if ((++spins & 1023u) == 0 && sh.abort_flag) break;
          if (spins > (1u << 28)) { sh.abort_flag = 1; break; }
        }
        if (sh.abort_flag) break;
        amax = fmaxf(amax, __uint_as_float(static_cast<unsigned>(seen)));
        const float scale = amax > 0.f ? amax * (1.0f / 448.0f) : 1.0f;
        const float inv = amax > 0.f ? 448.0f / amax : 1.0f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          int4 pk;
          unsigned *w = reinterpret_cast<unsigned *>(&pk);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float *v = acc + q * 16 + i * 4;
            const unsigned lo = __nv_cvt_float2_to_fp8x2(make_float2(v[0] * inv, v[1] * inv), __NV_SATFINITE, __NV_E4M3);
            const unsigned hi = __nv_cvt_float2_to_fp8x2(make_float2(v[2] * inv, v[3] * inv), __NV_SATFINITE, __NV_E4M3);
            w[i] = lo | (hi << 16);
          }
          *reinterpret_cast<int4 *>(stg + lane * EPI_ROW_BYTES + q * 16) = pk;
        }
        if (half == 0 && row_ok) *epi.scale_ptr(t, row) = scale;
        __syncwarp();
        // 64 bytes per row: 4 lanes per row, 8 rows per instruction.
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int r = it * 8 + lane / 4, seg = lane % 4;
          const int orow = quarter * 32 + r;
          if (orow < t.rows) {
            unsigned char *dst = epi.q_row_ptr(t, orow) + col0 + seg * 16;
            *reinterpret_cast<int4 *>(dst) = *reinterpret_cast<const int4 *>(stg + r * EPI_ROW_BYTES + seg * 16);
          }
        }
        __syncwarp();
      } else {
      // Write-out through the warp's padded staging rows, 32 columns at a time: 4 lanes per row write 64
      // contiguous bytes, 8 rows per instruction (instead of one row per thread in 16-byte pieces).
#pragma unroll
      for (int c = 0; c < OUT / 32; ++c) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          int4 pk;
          __nv_bfloat162 *p2 = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
          for (int i = 0; i < 4; ++i) p2[i] = __floats2bfloat162_rn(acc[c * 32 + q * 8 + 2 * i], acc[c * 32 + q * 8 + 2 * i + 1]);
          *reinterpret_cast<int4 *>(stg + lane * EPI_ROW_BYTES + q * 16) = pk;
        }
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int r = it * 8 + lane / 4, seg = lane % 4;
          const int orow = quarter * 32 + r;
          const int col = col0 + c * 32 + seg * 8;
          if (orow < t.rows && col < t.cols) {
            __nv_bfloat16 *out = epi.row_ptr(t, orow);
            if (out != nullptr) {
              const unsigned char *src = stg + r * EPI_ROW_BYTES + seg * 16;
              __nv_bfloat16 *dst = out + col;
              if (col + 8 <= t.cols && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
                if (EPI_ADD) sm100::red_add_bf16x8(dst, *reinterpret_cast<const int4 *>(src));
                else *reinterpret_cast<int4 *>(dst) = *reinterpret_cast<const int4 *>(src);
              } else {
                const __nv_bfloat16 *s16 = reinterpret_cast<const __nv_bfloat16 *>(src);
                for (int i = 0; i < 8 && col + i < t.cols; ++i) {
                  if (EPI_ADD) atomicAdd(dst + i, s16[i]);
                  else dst[i] = s16[i];
                }
              }
            }
          }
        }
        __syncwarp();
      }
      }
    }
  }
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
  if (warp == 1) {
    sm100::tcgen05_fence_after();
    sm100::tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && sh.abort_flag) atomicAdd(&gemm::g_gemm_errors, 1u);
}

}  // namespace gemm8
}  // namespace kernels
}  // namespace rocshmem
