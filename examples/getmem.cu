// Every PE reads a block of integers from its right-hand neighbour with a block-scope get.
// Counterpart of examples/rocshmem_getmem_test.cc in the reference.
//
//   python -m torch.distributed.run --no-python --nproc-per-node 2 --master-addr 127.0.0.1 ./getmem
#include <vector>

#include "common.h"

using namespace rocshmem;

__global__ void get_from_neighbour(int *dest, const int *source, size_t n) {
  rocshmem_wg_init();
  const int pe = (rocshmem_my_pe() + 1) % rocshmem_n_pes();
  rocshmem_int_get_wg(dest, source, n, pe);  // returns when the data is in dest
  rocshmem_wg_finalize();
}

int main() {
  select_device();
  rocshmem_init();
  const int me = rocshmem_my_pe(), npes = rocshmem_n_pes();
  const size_t n = 1 << 20;
  int *source = symmetric_alloc<int>(n), *dest = symmetric_alloc<int>(n);
  std::vector<int> host(n);
  for (size_t i = 0; i < n; ++i) host[i] = me * 1000003 + static_cast<int>(i);
  rocshmemx_heap_write(source, host.data(), n * sizeof(int));
  rocshmem_barrier_all();  // every source is filled

  get_from_neighbour<<<1, 1024>>>(dest, source, n);
  CHECK_CUDA(cudaGetLastError());
  CHECK_CUDA(cudaDeviceSynchronize());

  rocshmemx_heap_read(host.data(), dest, n * sizeof(int));
  const int from = (me + 1) % npes;
  bool ok = true;
  for (size_t i = 0; i < n && ok; ++i) ok = host[i] == from * 1000003 + static_cast<int>(i);
  rocshmem_barrier_all();
  rocshmem_free(dest);
  rocshmem_free(source);
  const int rc = report("getmem", ok);
  rocshmem_finalize();
  return rc;
}
