"""Debug checks (ROCSHMEM_DEBUG_CHECKS=1): a device call with a PE outside the job or an address outside the
symmetric heap is skipped and recorded in the error record; nothing traps and the context stays usable."""
import pytest
import torch

pytestmark = pytest.mark.gpu

NPES = 2
RMA_PUT, SC_THREAD = 0, 0


@pytest.fixture(scope="module")
def env():
    import rocshmem_b200 as shm
    from rocshmem_b200 import _native
    if shm.is_initialized():
        shm.finalize()
    shm.init(n_local=NPES, heap_size="64M", ROCSHMEM_WAIT_TIMEOUT_MS=2000, ROCSHMEM_DEBUG_CHECKS=1)
    yield shm, _native.load_test_kernels()
    torch.cuda.synchronize()
    shm.finalize()


def test_legal_calls_record_nothing(env):
    shm, k = env
    src = shm.zeros(256, torch.uint8)
    dst = shm.zeros(256, torch.uint8)
    src.fill_(9)
    torch.cuda.synchronize()
    shm.clear_error()
    # the kernel reduces the shift modulo n_pes, so the target PE is legal
    k.rma(RMA_PUT, SC_THREAD, dst.data_ptr(), src.data_ptr(), 256, 5, 0, 32, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert shm.get_error()["count"] == 0
    shm.free(dst)
    shm.free(src)


def test_address_outside_the_heap_is_recorded_not_dereferenced(env):
    shm, k = env
    src = shm.zeros(256, torch.uint8)
    outside = torch.zeros(256, dtype=torch.uint8, device="cuda")   # valid memory, but not symmetric
    torch.cuda.synchronize()
    shm.clear_error()
    k.rma(RMA_PUT, SC_THREAD, outside.data_ptr(), src.data_ptr(), 256, 1, 0, 32, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    err = shm.get_error(0)
    assert err["count"] >= 1 and err["kind"] == 4, err            # ROCSHMEM_ERR_BAD_ADDRESS
    assert torch.all(outside == 0), "the put must have been skipped"
    shm.clear_error()
    # the context is still usable
    dst = shm.zeros(256, torch.uint8)
    src.fill_(3)
    torch.cuda.synchronize()
    k.rma(RMA_PUT, SC_THREAD, dst.data_ptr(), src.data_ptr(), 256, 1, 0, 32, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert shm.get_error()["count"] == 0
    assert torch.all(shm.local_view(dst, 1) == 3)
    shm.free(dst)
    shm.free(src)
