// tcgen05 / TMEM GEMM kernels for sm_100a and the fused GEMM + collective kernels built on them.
// Host-callable launchers (plain C++). All matrices are row-major; "B" is always given as [N, K]
// (the layout of a weight matrix [out_features, in_features]), so C = A * B^T.
//
// There is no GEMM in the reference; these kernels exist because the tensor-parallel and
// expert-parallel paths fuse a GEMM with the collective that feeds or drains it.
#pragma once

#include <cstddef>
#include <cstdint>

#include "rocshmem/rocshmem_common.h"

namespace rocshmem {
namespace kernels {

// C[M, N] (bf16) = A[M, K] (bf16) * B[N, K]^T (bf16), fp32 accumulation in TMEM.
// K must be a multiple of 8 (16-byte rows for TMA); M and N are arbitrary (edges are predicated).
// Returns 0, a cudaError_t, or -1 when the driver cannot encode tensor maps.
int gemm_bf16(const void *a, const void *b, void *c, int m, int n, int k, void *stream);

// Grouped GEMM over row groups that share K and N but have their own weights:
// for group g, C[offsets[g] : offsets[g+1], :] = A[offsets[g] : offsets[g+1], :] * B[g]^T, with
// B [groups, N, K]. `offsets` (groups + 1 ints) lives in device memory, so the row counts need not
// be known on the host (they come out of the MoE dispatch). `max_rows` bounds offsets[groups].
// With swiglu != 0, N must be even and the output is [rows, N / 2]:
// out[:, j] = silu(acc[:, j]) * acc[:, j + N/2]  (gate and up projections stacked in B).
// The same product with two CTAs per 256 x 256 tile (tcgen05 cta_group::2, clusters of two).
int gemm_bf16_pair(const void *a, const void *b, void *c, int m, int n, int k, void *stream);
int gemm_bf16_one_cta(const void *a, const void *b, void *c, int m, int n, int k, void *stream);
int grouped_gemm_bf16(const void *a, const void *b, void *c, const int *offsets, int groups, int max_rows,
                      int n, int k, int swiglu, void *stream);

// The grouped GEMM fed directly by the bf16 rows of an expert-parallel dispatch: position p of the grouped order
// (offsets as above) reads row row_index[p] of `a_rows` [*, K] (copied into shared memory with cp.async by extra
// producer warps). K must be a multiple of 64. Output as for grouped_gemm_bf16, in grouped order. (e4m3 rows are
// gathered by the block-scaled kernel below; de-quantising them inside a bf16 kernel's producer warps was measured
// slower than a separate gather pass.)
int grouped_gemm_bf16_gathered(const void *a_rows, const int *row_index, const void *b, void *c, const int *offsets,
                               int groups, int n, int k, int swiglu, void *stream);
// The grouped GEMM whose result rows are scaled and summed where they belong: y[row_index[p], :] += weights[p] *
// (A[p, :] * B[g]^T) for every position p of group g (weights == nullptr: 1). y [*, N] bf16 must hold zeros (or the
// values to add to) beforehand; sums of several positions into one row are packed bf16 reductions in L2, so the
// order of additions, and with it the last bit of the result, may differ between runs. N must be a multiple of 8.
int grouped_gemm_bf16_scatter_add(const void *a, const void *b, void *y, const int *offsets, const int *row_index,
                                  const float *weights, int groups, int max_rows, int n, int k, void *stream);

// Device-side status of the last GEMM launched by this process: 0 ok, otherwise the number of
// CTAs whose bounded wait expired (they released their TMEM and returned early).
int gemm_error_count();

// Block-scaled e4m3 GEMM: C[M, N] (bf16) = (A_q * a_scale) (B_q * b_scale)^T with a_scale [M, K / 128]
// (one fp32 per row and 128-element K block) and b_scale [N / 128, K / 128] (one per 128 x 128 block).
// K must be a multiple of 512 and N of 128. The grouped form multiplies rows offsets[g] .. offsets[g + 1]
// with B_q[g] ([groups * N, K], scales [groups * N / 128, K / 128]).
int gemm_fp8_blockscaled(const void *a_q, const float *a_scale, const void *b_q, const float *b_scale, void *c, int m,
                         int n, int k, void *stream);
int grouped_gemm_fp8_blockscaled(const void *a_q, const float *a_scale, const void *b_q, const float *b_scale, void *c,
                                 const int *offsets, int groups, int max_rows, int n, int k, int swiglu,
                                 void *stream);

// Block-scaled forms of the two MoE-specific grouped GEMMs. The first is the gate/up projection with SwiGLU whose
// result is quantised in the epilogue to the next GEMM's operand format: out_q [rows, n / 2] e4m3 with out_s
// [rows, n / 256] fp32 (one scale per 128 columns); n must be a multiple of 256. The second is the block-scaled
// grouped_gemm_bf16_scatter_add. With row_index != nullptr the first one gathers its A rows and their scales by
// index (position p reads row row_index[p] of a_q / a_scale, which then need not be in grouped order; max_rows
// bounds the source rows).
int grouped_gemm_fp8_swiglu_quant(const void *a_q, const float *a_scale, const int *row_index, const void *b_q,
                                   const float *b_scale, void *out_q, float *out_s, const int *offsets, int groups,
                                   int max_rows, int n, int k, void *stream);
int grouped_gemm_fp8_scatter_add(const void *a_q, const float *a_scale, const void *b_q, const float *b_scale, void *y,
                                 const int *offsets, const int *row_index, const float *weights, int groups,
                                 int max_rows, int n, int k, void *stream);

// Tensor-parallel fused kernels on the symmetric heap (fused_kernels.cu).
// All-gather -> GEMM: every rank holds x_shard [m_shard, K] (symmetric); computes
// C[n_ranks * m_shard, N] = concat_ranks(x_shard) * B^T with its local B [N, K]. `gathered` is a
// symmetric scratch [n_ranks * m_shard, K] into which every member pushes its shard; `flags` holds one
// 32-bit counter per 128-row block (symmetric, zero-initialised once), `epoch` increases by one per call.
int ag_gemm_bf16(rocshmem_team_t team, const void *x_shard, void *gathered, unsigned long long *flags,
                 const void *b, void *c, int m_shard, int n, int k, unsigned epoch, int swiglu, void *stream);
// GEMM -> reduce-scatter: partial[M, N] = A[M, K_local] * B[N, K_local]^T is produced tile by tile and
// every tile is stored into the staging buffer of the rank that owns its rows
// (`staging` symmetric [n_ranks][m_shard, N] bf16); the owner then sums the n_ranks contributions into
// out [m_shard, N]. M = n_ranks * m_shard. `grid_counter` is one zero-initialised u64 in device memory
// reserved for this operation, `epoch` increases by one per call (1, 2, ...).
int gemm_rs_bf16(rocshmem_team_t team, const void *a, const void *b, void *staging, void *out, int m_shard,
                 int n, int k, unsigned long long *grid_counter, unsigned epoch, void *stream);

// Block-scaled e4m3 forms of the two fused kernels. x_q [m_shard, K] e4m3 and x_s [m_shard, K / 128] fp32 are
// the rank's quantised shard; gathered_q / gathered_s are symmetric buffers for all n_ranks shards; b_q [N, K] with b_scale
// [N / 128, K / 128]. K must be a multiple of 512, N of 128 (256 with swiglu).
int ag_gemm_fp8(rocshmem_team_t team, const void *x_q, const float *x_s, void *gathered_q, float *gathered_s,
                unsigned long long *flags, const void *b_q, const float *b_scale, void *c, int m_shard, int n, int k,
                unsigned epoch, int swiglu, void *stream);
int gemm_rs_fp8(rocshmem_team_t team, const void *a_q, const float *a_scale, const void *b_q, const float *b_scale,
                void *staging, void *out, int m_shard, int n, int k, unsigned long long *grid_counter, unsigned epoch,
                void *stream);

}  // namespace kernels
}  // namespace rocshmem
