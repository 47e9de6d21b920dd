// Teams and team contexts: the world team is split into the even and the odd PEs; each team runs its own
// max-reduction from a device kernel on a context created from the team. With one PE the single team has one
// member. (The reference exercises the same calls in tests/functional_tests/team_reduction_tester.cpp.)
//
//   python -m torch.distributed.run --no-python --nproc-per-node 4 --master-addr 127.0.0.1 ./team_reduce
#include <vector>

#include "common.h"

using namespace rocshmem;

__global__ void team_max(rocshmem_team_t team, int *dest, const int *source, int n) {
  __shared__ rocshmem_ctx_t ctx;
  rocshmem_wg_init();
  rocshmem_wg_team_create_ctx(team, ROCSHMEM_CTX_WG_PRIVATE, &ctx);
  rocshmem_ctx_int_max_wg_reduce(ctx, team, dest, source, n);
  rocshmem_wg_ctx_destroy(&ctx);
  rocshmem_wg_finalize();
}

int main() {
  select_device();
  rocshmem_init();
  const int me = rocshmem_my_pe(), npes = rocshmem_n_pes();
  // Both splits are collective over the world team; a PE gets ROCSHMEM_TEAM_INVALID for the team it is not in.
  rocshmem_team_t even = ROCSHMEM_TEAM_INVALID, odd = ROCSHMEM_TEAM_INVALID;
  rocshmem_team_split_strided(ROCSHMEM_TEAM_WORLD, 0, 2, (npes + 1) / 2, nullptr, 0, &even);
  if (npes > 1) rocshmem_team_split_strided(ROCSHMEM_TEAM_WORLD, 1, 2, npes / 2, nullptr, 0, &odd);
  rocshmem_team_t mine = (me % 2 == 0) ? even : odd;
  const int n = 4096;
  int *source = symmetric_alloc<int>(n), *dest = symmetric_alloc<int>(n);
  std::vector<int> host(n);
  for (int i = 0; i < n; ++i) host[i] = (i % (me + 2)) * 10 + me;
  rocshmemx_heap_write(source, host.data(), n * sizeof(int));
  rocshmem_barrier_all();

  team_max<<<1, 256>>>(mine, dest, source, n);
  CHECK_CUDA(cudaGetLastError());
  CHECK_CUDA(cudaDeviceSynchronize());

  rocshmemx_heap_read(host.data(), dest, n * sizeof(int));
  bool ok = rocshmem_team_my_pe(mine) == me / 2 && rocshmem_team_translate_pe(mine, me / 2, ROCSHMEM_TEAM_WORLD) == me;
  for (int i = 0; i < n && ok; ++i) {
    int want = 0;
    for (int p = me % 2; p < npes; p += 2) want = std::max(want, (i % (p + 2)) * 10 + p);
    ok = host[i] == want;
  }
  rocshmem_barrier_all();
  rocshmem_free(dest);
  rocshmem_free(source);
  if (odd != ROCSHMEM_TEAM_INVALID) rocshmem_team_destroy(odd);
  if (even != ROCSHMEM_TEAM_INVALID) rocshmem_team_destroy(even);
  const int rc = report("team_reduce", ok);
  rocshmem_finalize();
  return rc;
}
