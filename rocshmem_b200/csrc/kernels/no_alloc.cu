// Allocation-free variant of the MoE expert-layout kernels: the per-expert cursor scratch lives in a
// fixed device array of this file instead of caller-provided memory. See no_alloc.h for the contract.
#include "no_alloc.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "ep_kernels.hpp"

namespace {

constexpr int kMaxDevices = 64;

// One cursor per local expert. In host code this name is only a stand-in for the device object: the
// address that kernels may use is obtained with cudaGetSymbolAddress, per device.
static __device__ __align__(256) int g_cursor_scratch[ROCSHMEM_B200_NOALLOC_MAX_EXPERTS];

std::mutex g_setup_mutex;
int *g_scratch_on_device[kMaxDevices] = {};

// First pass: exclusive prefix of the per-expert pair counts, and cleared cursors.
__global__ void noalloc_offsets_kernel(const int *recv_info, int n_ranks, int experts_per_rank, int *offsets,
                                       int *cursor) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < experts_per_rank; ++e) {
      offsets[e] = run;
      cursor[e] = 0;  // the array keeps the previous call's values
      run += recv_info[1 + 2 * n_ranks + e];
    }
    offsets[experts_per_rank] = run;
  }
}

// Second pass: every (row, k) pair that selects a local expert takes the next position of that expert.
// An expert index outside [0, experts_per_rank) (a caller whose experts_per_rank is smaller than the
// dispatcher's) is skipped: its cursor was not cleared by this call and may lie outside the array.
__global__ void noalloc_layout_kernel(const int *recv_meta, const int *recv_info, int n_ranks, int experts_per_rank,
                                      int top_k, const int *offsets, int *row_index, int *pair_k, int *cursor) {
  using rocshmem::kernels::EP_META_IDX;
  using rocshmem::kernels::EP_META_WORDS;
  for (int s = 0; s < n_ranks; ++s) {
    const int start = recv_info[1 + s], count = recv_info[1 + n_ranks + s];
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < count * top_k; i += gridDim.x * blockDim.x) {
      const int row = start + i / top_k, k = i % top_k;
      const int e = recv_meta[size_t(row) * EP_META_WORDS + EP_META_IDX + k];
      if (e >= 0 && e < experts_per_rank) {
        const int pos = offsets[e] + atomicAdd(&cursor[e], 1);
        row_index[pos] = row;
        pair_k[pos] = k;
      }
    }
  }
}

// Device address of the scratch array on the current device, looked up once per device.
int scratch_for_current_device(int **out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return ROCSHMEM_B200_NOALLOC_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_on_device[dev] == nullptr) {
    int *ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_cursor_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (ptr == nullptr) return static_cast<int>(cudaErrorInvalidSymbol);
    g_scratch_on_device[dev] = ptr;
  }
  *out = g_scratch_on_device[dev];
  return 0;
}

}  // namespace

extern "C" int rocshmem_b200_expert_layout_noalloc(const int *recv_meta, const int *recv_info, int n_ranks,
                                                   int experts_per_rank, int top_k, int *offsets, int *row_index,
                                                   int *pair_k, void *stream_v) {
  if (recv_meta == nullptr || recv_info == nullptr || offsets == nullptr || row_index == nullptr || pair_k == nullptr ||
      n_ranks < 1 || experts_per_rank < 1 || top_k < 1) {
    return ROCSHMEM_B200_NOALLOC_BAD_ARGUMENT;
  }
  if (experts_per_rank > ROCSHMEM_B200_NOALLOC_MAX_EXPERTS || n_ranks > 64 || top_k > rocshmem::kernels::EP_MAX_TOPK) {
    std::fprintf(stderr,
                 "rocshmem_b200_expert_layout_noalloc: experts_per_rank=%d n_ranks=%d top_k=%d exceed the built-in "
                 "scratch (max %d experts per rank, 64 ranks, top-%d); use ep_expert_layout with caller scratch\n",
                 experts_per_rank, n_ranks, top_k, ROCSHMEM_B200_NOALLOC_MAX_EXPERTS, rocshmem::kernels::EP_MAX_TOPK);
    return ROCSHMEM_B200_NOALLOC_TOO_LARGE;
  }
  int *cursor = nullptr;
  if (int rc = scratch_for_current_device(&cursor)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  noalloc_offsets_kernel<<<1, 32, 0, stream>>>(recv_info, n_ranks, experts_per_rank, offsets, cursor);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const unsigned blocks = sms > 0 ? static_cast<unsigned>(sms) : 1u;
  noalloc_layout_kernel<<<blocks, 256, 0, stream>>>(recv_meta, recv_info, n_ranks, experts_per_rank, top_k, offsets,
                                                    row_index, pair_k, cursor);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
