// Team broadcast from a device kernel: the root's buffer reaches every other member of the world team.
// Counterpart of examples/rocshmem_broadcast_test.cc.
//
//   python -m torch.distributed.run --no-python --nproc-per-node 2 --master-addr 127.0.0.1 ./broadcast
#include <vector>

#include "common.h"

using namespace rocshmem;

__global__ void bcast(rocshmem_team_t team, int *dest, const int *source, size_t n, int root) {
  __shared__ rocshmem_ctx_t ctx;
  rocshmem_wg_init();
  rocshmem_wg_ctx_create(ROCSHMEM_CTX_WG_PRIVATE, &ctx);
  rocshmem_ctx_int_wg_broadcast(ctx, team, dest, source, static_cast<int>(n), root);
  rocshmem_ctx_quiet(ctx);
  rocshmem_wg_ctx_destroy(&ctx);
  rocshmem_wg_finalize();
}

int main() {
  select_device();
  rocshmem_init();
  const int me = rocshmem_my_pe();
  const size_t n = 100000;
  const int root = 0;
  int *source = symmetric_alloc<int>(n), *dest = symmetric_alloc<int>(n);
  std::vector<int> host(n);
  for (size_t i = 0; i < n; ++i) host[i] = me == root ? static_cast<int>(i) * 3 + 1 : -1;
  rocshmemx_heap_write(source, host.data(), n * sizeof(int));
  std::vector<int> zeros(n, 0);
  rocshmemx_heap_write(dest, zeros.data(), n * sizeof(int));
  rocshmem_barrier_all();

  bcast<<<1, 512>>>(ROCSHMEM_TEAM_WORLD, dest, source, n, root);
  CHECK_CUDA(cudaGetLastError());
  CHECK_CUDA(cudaDeviceSynchronize());

  rocshmemx_heap_read(host.data(), dest, n * sizeof(int));
  bool ok = true;
  // The root's dest is not written by a broadcast.
  for (size_t i = 0; i < n && ok; ++i) ok = host[i] == (me == root ? 0 : static_cast<int>(i) * 3 + 1);
  rocshmem_barrier_all();
  rocshmem_free(dest);
  rocshmem_free(source);
  const int rc = report("broadcast", ok);
  rocshmem_finalize();
  return rc;
}
