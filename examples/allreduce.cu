// Sum-allreduce of floats, twice: from a device kernel with the block-collective API, and from the
// host with the stream-ordered library kernel (which picks one-shot, two-shot or NVLS by size).
// Counterpart of examples/rocshmem_allreduce_test.cc.
//
//   python -m torch.distributed.run --no-python --nproc-per-node 2 --master-addr 127.0.0.1 ./allreduce
#include <cmath>
#include <vector>

#include "common.h"

using namespace rocshmem;

__global__ void reduce_in_kernel(rocshmem_team_t team, float *dest, const float *source, int n) {
  __shared__ rocshmem_ctx_t ctx;
  rocshmem_wg_init();
  rocshmem_wg_ctx_create(ROCSHMEM_CTX_WG_PRIVATE, &ctx);
  rocshmem_ctx_float_sum_wg_reduce(ctx, team, dest, source, n);
  rocshmem_wg_ctx_destroy(&ctx);
  rocshmem_wg_finalize();
}

static bool check(const float *heap, size_t n, int npes) {
  std::vector<float> host(n);
  rocshmemx_heap_read(host.data(), heap, n * sizeof(float));
  const float pes = static_cast<float>(npes);
  for (size_t i = 0; i < n; ++i) {
    // sum over p of (p + 1) * (i % 97): exact in fp32 for these magnitudes
    const float want = pes * (pes + 1) / 2 * static_cast<float>(i % 97);
    if (std::fabs(host[i] - want) > 1e-3f * (1 + want)) return false;
  }
  return true;
}

int main() {
  select_device();
  rocshmem_init();
  const int me = rocshmem_my_pe(), npes = rocshmem_n_pes();
  const size_t n = 1 << 18;
  float *source = symmetric_alloc<float>(n), *dest = symmetric_alloc<float>(n);
  std::vector<float> host(n);
  for (size_t i = 0; i < n; ++i) host[i] = static_cast<float>(me + 1) * static_cast<float>(i % 97);
  rocshmemx_heap_write(source, host.data(), n * sizeof(float));
  rocshmem_barrier_all();

  reduce_in_kernel<<<1, 1024>>>(ROCSHMEM_TEAM_WORLD, dest, source, static_cast<int>(n));
  CHECK_CUDA(cudaGetLastError());
  CHECK_CUDA(cudaDeviceSynchronize());
  bool ok = check(dest, n, npes);

  std::vector<float> zeros(n, 0.f);
  rocshmemx_heap_write(dest, zeros.data(), n * sizeof(float));
  rocshmem_barrier_all();
  const int rc_host = rocshmem_ctx_float_sum_reduce(ROCSHMEM_CTX_DEFAULT, ROCSHMEM_TEAM_WORLD, dest, source, static_cast<int>(n));
  ok = ok && rc_host == 0 && check(dest, n, npes);

  rocshmem_barrier_all();
  rocshmem_free(dest);
  rocshmem_free(source);
  const int rc = report("allreduce", ok);
  rocshmem_finalize();
  return rc;
}
