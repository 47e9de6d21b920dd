// Host-callable launchers of the MoE feed-forward glue kernels (see moe_kernels.cu). All pointers are
// device addresses on the current device; every call is stream-ordered and returns 0 or a CUDA error.
#pragma once

namespace rocshmem {
namespace kernels {

// out[pos, :] = row row_index[pos] of the receive buffer as bf16, for pos < offsets[experts].
// fp8 != 0: recv_x holds e4m3 bytes with one fp32 scale per 128 elements; else bf16 rows.
int moe_gather_rows(const void *recv_x, const float *recv_scales, int fp8, const int *offsets, int experts,
                    const int *row_index, int hidden, void *out_bf16, void *stream);

// Zeroes the rows of y [*, hidden] (bf16) that recv_info lists as received (the destination of a scatter-add
// grouped GEMM must start from zero).
int moe_zero_rows(const int *recv_info, int n_ranks, int hidden, void *y_bf16, void *stream);

}  // namespace kernels
}  // namespace rocshmem
