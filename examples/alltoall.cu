// Team all-to-all from a device kernel: chunk j of every PE's source lands as chunk "sender" of PE
// j's dest. Counterpart of examples/rocshmem_alltoall_test.cc.
//
//   python -m torch.distributed.run --no-python --nproc-per-node 2 --master-addr 127.0.0.1 ./alltoall
#include <vector>

#include "common.h"

using namespace rocshmem;

__global__ void exchange(rocshmem_team_t team, long *dest, const long *source, int nelems) {
  __shared__ rocshmem_ctx_t ctx;
  rocshmem_wg_init();
  rocshmem_wg_team_create_ctx(team, ROCSHMEM_CTX_WG_PRIVATE, &ctx);
  rocshmem_ctx_long_wg_alltoall(ctx, team, dest, source, nelems);
  rocshmem_wg_ctx_destroy(&ctx);
  rocshmem_wg_finalize();
}

int main() {
  select_device();
  rocshmem_init();
  const int me = rocshmem_my_pe(), npes = rocshmem_n_pes();
  const int nelems = 8192;  // per destination
  long *source = symmetric_alloc<long>(size_t(nelems) * npes), *dest = symmetric_alloc<long>(size_t(nelems) * npes);
  std::vector<long> host(size_t(nelems) * npes);
  for (int j = 0; j < npes; ++j) {
    for (int i = 0; i < nelems; ++i) host[size_t(j) * nelems + i] = (long(me) << 40) | (long(j) << 20) | i;
  }
  rocshmemx_heap_write(source, host.data(), host.size() * sizeof(long));
  rocshmem_barrier_all();

  exchange<<<1, 1024>>>(ROCSHMEM_TEAM_WORLD, dest, source, nelems);
  CHECK_CUDA(cudaGetLastError());
  CHECK_CUDA(cudaDeviceSynchronize());

  rocshmemx_heap_read(host.data(), dest, host.size() * sizeof(long));
  bool ok = true;
  for (int j = 0; j < npes && ok; ++j) {
    for (int i = 0; i < nelems && ok; ++i) ok = host[size_t(j) * nelems + i] == ((long(j) << 40) | (long(me) << 20) | i);
  }
  rocshmem_barrier_all();
  rocshmem_free(dest);
  rocshmem_free(source);
  const int rc = report("alltoall", ok);
  rocshmem_finalize();
  return rc;
}
