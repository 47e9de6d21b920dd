// Helpers shared by the example programs.
#pragma once

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>

#include <rocshmem/rocshmem.h>

#define CHECK_CUDA(call)                                                                          \
  do {                                                                                            \
    cudaError_t e_ = (call);                                                                      \
    if (e_ != cudaSuccess) {                                                                      \
      std::fprintf(stderr, "%s:%d: %s\n", __FILE__, __LINE__, cudaGetErrorString(e_));            \
      rocshmem::rocshmem_global_exit(1);                                                          \
    }                                                                                             \
  } while (0)

// One GPU per PE: my_pe() is usable before init (it reads RANK), as in the reference's examples
// (examples/rocshmem_allreduce_test.cc:75-83).
inline void select_device() {
  int count = 0;
  CHECK_CUDA(cudaGetDeviceCount(&count));
  CHECK_CUDA(cudaSetDevice(rocshmem::rocshmem_my_pe() % count));
}

template <typename T>
T *symmetric_alloc(size_t n) {
  T *p = static_cast<T *>(rocshmem::rocshmem_malloc(n * sizeof(T)));
  if (p == nullptr) {
    std::fprintf(stderr, "PE %d: rocshmem_malloc of %zu bytes failed\n", rocshmem::rocshmem_my_pe(), n * sizeof(T));
    rocshmem::rocshmem_global_exit(1);
  }
  return p;
}

inline int report(const char *name, bool ok) {
  std::printf("[PE %d] %s: %s\n", rocshmem::rocshmem_my_pe(), name, ok ? "PASS" : "FAIL");
  return ok ? 0 : 1;
}
