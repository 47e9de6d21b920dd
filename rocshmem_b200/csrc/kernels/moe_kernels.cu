// Glue between the expert-parallel dispatch / combine and the grouped GEMMs of a MoE feed-forward layer:
//   moe_gather_rows     received rows -> expert-sorted bf16 rows (de-quantising 1x128 block-scaled e4m3); used when
//                       e4m3 rows feed bf16 experts (the block-scaled experts gather inside their GEMM)
//   moe_zero_rows       clears the result rows that the down projection's scatter-add epilogue accumulates into
// All sizes that depend on the routing (pair count, row ranges) are read on the device, so the layer runs
// without a host synchronisation. One PE per process; pointers are plain device addresses.
//
// No counterpart exists in the reference.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "ep_kernels.hpp"
#include "launch.cuh"
#include "moe_kernels.hpp"

namespace rocshmem {
namespace kernels {

namespace {

constexpr int kThreads = 256;

// One warp per expert-sorted position. fp8: a lane de-quantises 16 elements per step (one 16-byte load,
// two 16-byte stores); 8 lanes share a scale.
template <bool FP8>
__global__ void gather_rows_kernel(const void *recv_x, const float *recv_scales, const int *offsets, int experts,
                                   const int *row_index, int hidden, __nv_bfloat16 *out) {
  const int total = offsets[experts];
  const int lane = threadIdx.x % 32;
  const int warps = gridDim.x * (blockDim.x / 32);
  for (int pos = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32; pos < total; pos += warps) {
    const int row = row_index[pos];
    __nv_bfloat16 *dst = out + size_t(pos) * hidden;
    if (FP8) {
      const uint8_t *src = static_cast<const uint8_t *>(recv_x) + size_t(row) * hidden;
      const float *sc = recv_scales + size_t(row) * (hidden / 128);
      for (int c = lane * 16; c < hidden; c += 32 * 16) {
        const int4 raw = *reinterpret_cast<const int4 *>(src + c);
        const float s = sc[c / 128];
        const __nv_fp8x2_storage_t *p2 = reinterpret_cast<const __nv_fp8x2_storage_t *>(&raw);
        int4 o[2];
        __nv_bfloat162 *o2 = reinterpret_cast<__nv_bfloat162 *>(o);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(p2[i], __NV_E4M3);
          const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&h));
          o2[i] = __floats2bfloat162_rn(f.x * s, f.y * s);
        }
        reinterpret_cast<int4 *>(dst + c)[0] = o[0];
        reinterpret_cast<int4 *>(dst + c)[1] = o[1];
      }
    } else {
      const int4 *src = reinterpret_cast<const int4 *>(static_cast<const __nv_bfloat16 *>(recv_x) + size_t(row) * hidden);
      for (int v = lane; v < hidden / 8; v += 32) reinterpret_cast<int4 *>(dst)[v] = src[v];
    }
  }
}

// Zeroes the received rows listed in recv_info (16 bytes per thread and step).
__global__ void zero_rows_kernel(const int *recv_info, int n_ranks, int hidden, __nv_bfloat16 *y) {
  const size_t vec_per_row = size_t(hidden) / 8;
  for (int s = 0; s < n_ranks; ++s) {
    const size_t first = recv_info[1 + s], count = recv_info[1 + n_ranks + s];
    int4 *base = reinterpret_cast<int4 *>(y + first * hidden);
    const size_t total = count * vec_per_row;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
      base[i] = make_int4(0, 0, 0, 0);
    }
  }
}

}  // namespace

int moe_zero_rows(const int *recv_info, int n_ranks, int hidden, void *y_bf16, void *stream) {
  if (hidden <= 0 || hidden % 8 || n_ranks < 1) return cudaErrorInvalidValue;
  zero_rows_kernel<<<static_cast<unsigned>(device_sm_count() * 4), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      recv_info, n_ranks, hidden, static_cast<__nv_bfloat16 *>(y_bf16));
  return cudaGetLastError();
}

int moe_gather_rows(const void *recv_x, const float *recv_scales, int fp8, const int *offsets, int experts,
                    const int *row_index, int hidden, void *out_bf16, void *stream) {
  if (hidden <= 0 || (fp8 ? hidden % 512 : hidden % 8) || experts < 1) return cudaErrorInvalidValue;
  const unsigned blocks = static_cast<unsigned>(device_sm_count() * 4);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (fp8) {
    gather_rows_kernel<true><<<blocks, kThreads, 0, s>>>(recv_x, recv_scales, offsets, experts, row_index, hidden,
                                                         static_cast<__nv_bfloat16 *>(out_bf16));
  } else {
    gather_rows_kernel<false><<<blocks, kThreads, 0, s>>>(recv_x, recv_scales, offsets, experts, row_index, hidden,
                                                          static_cast<__nv_bfloat16 *>(out_bf16));
  }
  return cudaGetLastError();
}

}  // namespace kernels
}  // namespace rocshmem
