"""Model blocks on one GPU (a team of one PE): the whole kernel chain of each layer runs, only the
NVLink hops are local. Compared against plain PyTorch fp32 evaluations of the same layers."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def shm():
    import rocshmem_b200 as s
    if s.is_initialized():
        s.finalize()
    s.init(n_local=1, heap_size="2G", ROCSHMEM_WAIT_TIMEOUT_MS=5000)
    yield s
    torch.cuda.synchronize()
    s.finalize()


def clean(shm):
    torch.cuda.synchronize()
    err = shm.get_error(0)
    assert err["count"] == 0, err


@pytest.mark.parametrize("quantize", [True, False])
@pytest.mark.parametrize("E,K,H,I,T", [(8, 2, 1024, 512, 200), (16, 8, 2048, 256, 333)])
def test_moe_feed_forward(shm, quantize, E, K, H, I, T):
    """bf16 experts: behind a quantised dispatch (rows de-quantised into expert order by one kernel) and behind a bf16
    dispatch (rows gathered inside the GEMM)."""
    from rocshmem_b200.models import moe_ffn
    from rocshmem_b200.ops import gemm, moe
    layer = moe_ffn.MoEFeedForward(E, K, H, I, max_tokens=T + 5, quantize=quantize, seed=2, fp8_experts=False)
    for rep in range(2):
        x = torch.randn(T, H, generator=torch.Generator().manual_seed(rep + 1)).to(torch.bfloat16)
        idx, w = moe.make_routing(T, E, K, seed=50 + rep)
        if rep:
            idx[::6, -1] = -1
        before = gemm.gemm_error_count()
        out = layer(x.cuda(), idx.cuda(), w.cuda())
        clean(shm)
        assert gemm.gemm_error_count() == before
        want = moe_ffn.reference_forward(x, idx, w, H, I, seed=2, quantize=quantize)
        err = (out.float().cpu() - want).abs().max().item()
        assert err <= 3e-2 * want.abs().max().item() + 0.02, (rep, err, want.abs().max().item())
    layer.destroy()


@pytest.mark.parametrize("d_model,d_ff,m", [(1024, 512, 256), (2048, 1280, 384)])
def test_tp_mlp_single_rank(shm, d_model, d_ff, m):
    from rocshmem_b200.models import tp_mlp
    from rocshmem_b200.ops import gemm
    mlp = tp_mlp.TensorParallelMLP(d_model, d_ff, m, seed=4)
    x = (torch.randn(m, d_model, generator=torch.Generator().manual_seed(9)) * 0.5).to(torch.bfloat16)
    want = tp_mlp.reference_forward(x, 1, d_model, d_ff, seed=4)
    for rep in range(2):
        before = gemm.gemm_error_count()
        out = mlp(x.cuda())
        clean(shm)
        assert gemm.gemm_error_count() == before
        err = (out.float().cpu() - want).abs().max().item()
        assert err <= 2e-2 * want.abs().max().item() + 0.05, (rep, err)


def test_moe_feed_forward_fp8_experts(shm):
    """e4m3 rows from the dispatch feed block-scaled fp8 grouped GEMMs directly (the default where shapes allow)."""
    from rocshmem_b200.models import moe_ffn
    from rocshmem_b200.ops import gemm, moe
    E, K, H, I, T = 8, 2, 1024, 512, 300
    layer = moe_ffn.MoEFeedForward(E, K, H, I, max_tokens=T, seed=6)
    assert layer.fp8_experts
    for rep in range(2):
        x = torch.randn(T, H, generator=torch.Generator().manual_seed(rep + 20)).to(torch.bfloat16)
        idx, w = moe.make_routing(T, E, K, seed=70 + rep)
        before = gemm.gemm_error_count()
        out = layer(x.cuda(), idx.cuda(), w.cuda())
        clean(shm)
        assert gemm.gemm_error_count() == before
        want = moe_ffn.reference_forward(x, idx, w, H, I, seed=6, fp8_experts=True)
        err = (out.float().cpu() - want).abs().max().item()
        # the hidden activation is re-quantised from slightly different bf16 values than the reference's
        assert err <= 5e-2 * want.abs().max().item() + 0.03, (rep, err, want.abs().max().item())


@pytest.mark.parametrize("d_model,d_ff,m", [(1024, 512, 256), (2048, 1536, 384)])
def test_tp_mlp_fp8_single_rank(shm, d_model, d_ff, m):
    from rocshmem_b200.models import tp_mlp
    from rocshmem_b200.ops import gemm
    mlp = tp_mlp.TensorParallelMLPFp8(d_model, d_ff, m, seed=4)
    x = (torch.randn(m, d_model, generator=torch.Generator().manual_seed(9)) * 0.5).to(torch.bfloat16)
    want = tp_mlp.reference_forward_fp8(x, 1, d_model, d_ff, seed=4)
    for rep in range(2):
        before = gemm.gemm_error_count()
        out = mlp(x.cuda())
        clean(shm)
        assert gemm.gemm_error_count() == before
        err = (out.float().cpu() - want).abs().max().item()
        assert err <= 5e-2 * want.abs().max().item() + 0.05, (rep, err)
