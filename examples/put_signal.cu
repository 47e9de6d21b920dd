// Ring of put-with-signal: PE i sends a message to PE i + 1 together with a signal update, and
// waits for the signal of its own incoming message before checking it. No barrier is involved:
// the signal alone orders the data. Counterpart of examples/rocshmem_put_signal_test.cc.
//
//   python -m torch.distributed.run --no-python --nproc-per-node 2 --master-addr 127.0.0.1 ./put_signal
#include <vector>

#include "common.h"

using namespace rocshmem;

__global__ void ring(uint64_t *message, const uint64_t *payload, size_t n, uint64_t *signal, int *arrived_ok) {
  rocshmem_wg_init();
  const int me = rocshmem_my_pe(), npes = rocshmem_n_pes();
  rocshmem_ulong_put_signal_wg(reinterpret_cast<unsigned long *>(message),
                               reinterpret_cast<const unsigned long *>(payload), n, signal, 1,
                               ROCSHMEM_SIGNAL_ADD, (me + 1) % npes);
  if (threadIdx.x == 0) {
    rocshmem_uint64_wait_until(signal, ROCSHMEM_CMP_EQ, 1);  // bounded: reports through the error record
    const uint64_t from = static_cast<uint64_t>((me + npes - 1) % npes);
    int ok = rocshmem_signal_fetch(signal) == 1;
    for (size_t i = 0; i < n; ++i) ok &= message[i] == (from << 32 | i);
    *arrived_ok = ok;
  }
  __syncthreads();
  rocshmem_wg_finalize();
}

int main() {
  select_device();
  rocshmem_init();
  const int me = rocshmem_my_pe();
  const size_t n = 4096;
  uint64_t *payload = symmetric_alloc<uint64_t>(n), *message = symmetric_alloc<uint64_t>(n);
  uint64_t *signal = symmetric_alloc<uint64_t>(1);
  std::vector<uint64_t> host(n);
  for (size_t i = 0; i < n; ++i) host[i] = static_cast<uint64_t>(me) << 32 | i;
  rocshmemx_heap_write(payload, host.data(), n * sizeof(uint64_t));
  const uint64_t zero = 0;
  rocshmemx_heap_write(signal, &zero, sizeof(zero));
  int *flag = nullptr;
  CHECK_CUDA(cudaMalloc(&flag, sizeof(int)));
  CHECK_CUDA(cudaMemset(flag, 0, sizeof(int)));
  rocshmem_barrier_all();  // signals are zero everywhere before anybody sends

  ring<<<1, 256>>>(message, payload, n, signal, flag);
  CHECK_CUDA(cudaGetLastError());
  CHECK_CUDA(cudaDeviceSynchronize());

  int ok = 0;
  CHECK_CUDA(cudaMemcpy(&ok, flag, sizeof(int), cudaMemcpyDeviceToHost));
  const rocshmem_error_record err = rocshmemx_get_error();
  rocshmem_barrier_all();
  cudaFree(flag);
  rocshmem_free(signal);
  rocshmem_free(message);
  rocshmem_free(payload);
  const int rc = report("put_signal", ok == 1 && err.kind == 0);
  rocshmem_finalize();
  return rc;
}
