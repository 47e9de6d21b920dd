// Kernel launch helper aware of "several PEs per process": with one PE per process a kernel is
// launched normally with gridDim.z == 1; otherwise it is launched once, cooperatively, with
// gridDim.z == n_local so that the PEs (which wait on one another) are guaranteed to be co-resident.
#pragma once

#include <cuda_runtime.h>

#include <algorithm>

#include "../runtime/runtime.hpp"

namespace rocshmem {
namespace kernels {

inline int device_sm_count() {
  static int sms = [] {
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n > 0 ? n : 1;
  }();
  return sms;
}

// Largest blocks-per-PE count for which all PEs' blocks of `kernel` fit on the GPU at once.
template <typename K>
inline unsigned coresident_blocks_per_pe(K kernel, unsigned threads, size_t smem, int n_local) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, static_cast<int>(threads), smem) !=
          cudaSuccess || per_sm < 1) {
    cudaGetLastError();
    per_sm = 1;
  }
  long total = static_cast<long>(per_sm) * device_sm_count();
  return static_cast<unsigned>(std::max<long>(1, total / std::max(1, n_local)));
}

// `cooperative`: blocks of one PE wait for each other inside the kernel (grid barrier), so
// co-residency is required even with one PE per process.
template <typename T>
struct same_as_kernel { using type = T; };

// Arguments are converted to the kernel's exact parameter types before their addresses are taken.
template <typename... KArgs>
inline cudaError_t launch_pes(void (*kernel)(KArgs...), unsigned blocks, unsigned threads, size_t smem,
                              cudaStream_t stream, bool cooperative,
                              typename same_as_kernel<KArgs>::type... args) {
  Runtime &rt = Runtime::instance();
  const int n_local = rt.n_local();
  dim3 grid(blocks, 1, static_cast<unsigned>(n_local));
  dim3 block(threads, 1, 1);
  if (n_local > 1 || cooperative) {
    unsigned fit = coresident_blocks_per_pe(kernel, threads, smem, n_local);
    if (blocks > fit) return cudaErrorCooperativeLaunchTooLarge;
    void *params[] = {const_cast<void *>(static_cast<const void *>(&args))...};
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(kernel), grid, block, params,
                                       smem, stream);
  }
  kernel<<<grid, block, smem, stream>>>(args...);
  return cudaGetLastError();
}

}  // namespace kernels
}  // namespace rocshmem
