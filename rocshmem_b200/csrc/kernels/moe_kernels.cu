// Glue between the expert-parallel dispatch / combine and the grouped GEMMs of a MoE feed-forward layer:
//   moe_gather_rows     received rows -> expert-sorted bf16 rows (de-quantising 1x128 block-scaled e4m3)
//   moe_inverse_map     position of every (row, k) pair in the expert-sorted order
//   moe_reduce_pairs    expert outputs -> one bf16 row per received row, sum over the row's local experts
//                       weighted by the gate weights carried in the row's metadata record
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

__global__ void inverse_map_kernel(const int *offsets, int experts, const int *row_index, const int *pair_k,
                                   int top_k, int *inverse) {
  const int total = offsets[experts];
  for (int pos = blockIdx.x * blockDim.x + threadIdx.x; pos < total; pos += gridDim.x * blockDim.x) {
    inverse[row_index[pos] * top_k + pair_k[pos]] = pos;
  }
}

// One warp per received row: y[row] = sum over k with a local expert of w[row, k] * pairs[inverse[row, k]].
__global__ void reduce_pairs_kernel(const __nv_bfloat16 *pairs, const int *inverse, const int *recv_meta,
                                    const int *recv_info, int n_ranks, int top_k, int hidden, int weighted,
                                    __nv_bfloat16 *y) {
  const int lane = threadIdx.x % 32;
  const int warps = gridDim.x * (blockDim.x / 32);
  const int warp = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  for (int s = 0; s < n_ranks; ++s) {
    const int first = recv_info[1 + s], count = recv_info[1 + n_ranks + s];
    for (int r = warp; r < count; r += warps) {
      const int row = first + r;
      const int *meta = recv_meta + size_t(row) * EP_META_WORDS;
      int pos[EP_MAX_TOPK];
      float w[EP_MAX_TOPK];
#pragma unroll
      for (int k = 0; k < EP_MAX_TOPK; ++k) {
        const bool live = k < top_k && meta[EP_META_IDX + k] >= 0;
        pos[k] = live ? inverse[row * top_k + k] : -1;
        w[k] = live ? (weighted ? __int_as_float(meta[EP_META_WEIGHT + k]) : 1.0f) : 0.f;
      }
      // Two 16-byte columns per lane and step: twice the loads in flight (the kernel is latency-bound,
      // a row has one or two live sources on average).
      const int nvec = hidden / 8;
      for (int v0 = lane; v0 < nvec; v0 += 64) {
        const int v1 = v0 + 32;
        const bool two = v1 < nvec;
        float acc[2][8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[0][i] = acc[1][i] = 0.f;
        int4 raw[2][EP_MAX_TOPK];
#pragma unroll
        for (int k = 0; k < EP_MAX_TOPK; ++k) {
          if (pos[k] >= 0) {
            const int4 *src = reinterpret_cast<const int4 *>(pairs + size_t(pos[k]) * hidden);
            raw[0][k] = src[v0];
            if (two) raw[1][k] = src[v1];
          }
        }
#pragma unroll
        for (int k = 0; k < EP_MAX_TOPK; ++k) {
          if (pos[k] >= 0) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              if (u == 1 && !two) continue;
              const __nv_bfloat162 *p2 = reinterpret_cast<const __nv_bfloat162 *>(&raw[u][k]);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(p2[i]);
                acc[u][2 * i] += w[k] * f.x;
                acc[u][2 * i + 1] += w[k] * f.y;
              }
            }
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (u == 1 && !two) continue;
          int4 o;
          __nv_bfloat162 *o2 = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
          for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(acc[u][2 * i], acc[u][2 * i + 1]);
          reinterpret_cast<int4 *>(y + size_t(row) * hidden)[u ? v1 : v0] = o;
        }
      }
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

int moe_inverse_map(const int *offsets, int experts, const int *row_index, const int *pair_k, int top_k,
                    int *inverse, void *stream) {
  if (experts < 1 || top_k < 1 || top_k > EP_MAX_TOPK) return cudaErrorInvalidValue;
  inverse_map_kernel<<<static_cast<unsigned>(device_sm_count()), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      offsets, experts, row_index, pair_k, top_k, inverse);
  return cudaGetLastError();
}

int moe_reduce_pairs(const void *pairs_bf16, const int *inverse, const int *recv_meta, const int *recv_info,
                     int n_ranks, int top_k, int hidden, int weighted, void *y_bf16, void *stream) {
  if (hidden <= 0 || hidden % 8 || top_k < 1 || top_k > EP_MAX_TOPK || n_ranks < 1) return cudaErrorInvalidValue;
  reduce_pairs_kernel<<<static_cast<unsigned>(device_sm_count() * 4), kThreads, 0,
                        static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16 *>(pairs_bf16), inverse, recv_meta, recv_info, n_ranks, top_k, hidden, weighted,
      static_cast<__nv_bfloat16 *>(y_bf16));
  return cudaGetLastError();
}

}  // namespace kernels
}  // namespace rocshmem
