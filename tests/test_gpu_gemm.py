"""tcgen05 / TMEM GEMM kernels against plain PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def ref_gemm(a, b):
    return a.float() @ b.float().t()


def close(got, want, k):
    # bf16 output rounding (2^-8 relative) plus fp32 accumulation noise over k terms
    err = (got.float() - want).abs()
    tol = 1e-2 * want.abs() + 2e-2 * (k ** 0.5) * 0.02 + 1e-3
    return bool((err <= tol).all()), float(err.max())


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 128), (300, 520, 1024), (1024, 1024, 4096),
                                   (64, 8, 256), (1000, 3584, 512)])
def test_gemm_bf16(m, n, k):
    from rocshmem_b200.ops import gemm
    g = torch.Generator(device="cuda").manual_seed(m * 7 + n)
    a = (torch.randn(m, k, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(n, k, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    before = gemm.gemm_error_count()
    c = gemm.gemm_bf16(a, b)
    torch.cuda.synchronize()
    assert gemm.gemm_error_count() == before, "a GEMM CTA hit its wait budget"
    ok, err = close(c, ref_gemm(a, b), k)
    assert ok, f"max abs error {err}"


def test_gemm_bf16_identity_pattern():
    """Exact check of the operand layout: B = identity picks columns of A."""
    from rocshmem_b200.ops import gemm
    m, k = 256, 512
    a = torch.arange(m * k, device="cuda").remainder(251).reshape(m, k).to(torch.bfloat16)
    b = torch.eye(k, device="cuda", dtype=torch.bfloat16)
    c = gemm.gemm_bf16(a, b)
    torch.cuda.synchronize()
    assert torch.equal(c, a)


@pytest.mark.parametrize("swiglu", [False, True])
def test_grouped_gemm(swiglu):
    from rocshmem_b200.ops import gemm
    groups, n, k = 5, 512, 768
    counts = [130, 0, 7, 256, 301]
    offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device="cuda")
    rows = sum(counts)
    g = torch.Generator(device="cuda").manual_seed(3)
    a = (torch.randn(rows + 40, k, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(groups, n, k, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
    width = n // 2 if swiglu else n
    out = torch.full((rows + 40, width), -7.0, dtype=torch.bfloat16, device="cuda")
    gemm.grouped_gemm_bf16(a, b, offsets, swiglu=swiglu, out=out)
    torch.cuda.synchronize()
    lo = 0
    for gi, cnt in enumerate(counts):
        if cnt:
            acc = ref_gemm(a[lo:lo + cnt], b[gi])
            want = torch.nn.functional.silu(acc[:, :n // 2]) * acc[:, n // 2:] if swiglu else acc
            ok, err = close(out[lo:lo + cnt], want, k)
            assert ok, f"group {gi}: max abs error {err}"
        lo += cnt
    assert torch.all(out[rows:] == -7.0)  # rows past the last group are untouched


def test_gemm_throughput_report(capsys):
    """Not an assertion on speed: prints the achieved rate for the tensor-parallel MLP shape."""
    from rocshmem_b200.ops import gemm
    m, n, k = 8192, 3584, 8192
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    b = torch.randn(n, k, device="cuda").to(torch.bfloat16)
    c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    for _ in range(3):
        gemm.gemm_bf16(a, b, out=c)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(10):
        gemm.gemm_bf16(a, b, out=c)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / 10
    ref = torch.matmul(a[:256], b.t())
    assert torch.allclose(c[:256].float(), ref.float(), rtol=2e-2, atol=1.0)
    with capsys.disabled():
        print(f"\n[gemm_bf16 {m}x{n}x{k}] {ms * 1e3:.1f} us, {2 * m * n * k / ms / 1e9:.0f} TFLOP/s")
