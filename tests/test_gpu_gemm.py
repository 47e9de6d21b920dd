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
    # The whole result against an fp32 product (in row slabs to bound the reference's memory): the shape has
    # wave-quantised tails, several rasterisation groups and operands larger than L2.
    for lo in range(0, m, 2048):
        ok, err = close(c[lo:lo + 2048], ref_gemm(a[lo:lo + 2048], b), k)
        assert ok, f"rows {lo}..{lo + 2048}: max abs error {err}"
    with capsys.disabled():
        print(f"\n[gemm_bf16 {m}x{n}x{k}] {ms * 1e3:.1f} us, {2 * m * n * k / ms / 1e9:.0f} TFLOP/s")


# ---- block-scaled fp8 ---------------------------------------------------------------------------------------------

def _fp8_inputs(m, n, k, seed, groups=None):
    from rocshmem_b200.ops import gemm, moe
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = (torch.randn(m, k, generator=g, device="cuda") * torch.rand(m, 1, generator=g, device="cuda") * 2).to(torch.bfloat16)
    shape = (n, k) if groups is None else (groups, n, k)
    b = (torch.randn(*shape, generator=g, device="cuda") * 0.3).to(torch.bfloat16)
    a_q, a_s = moe.fp8_quantize_1x128(a)
    b_q, b_s = gemm.quantize_weight_128x128(b)
    a_deq = moe.ref_dequantize_1x128(a_q, a_s)
    b_deq = gemm.dequantize_weight_128x128(b_q, b_s)
    return a_q, a_s, b_q, b_s, a_deq, b_deq


@pytest.mark.parametrize("m,n,k", [(128, 256, 512), (300, 384, 1024), (1024, 1280, 2048), (77, 128, 3584)])
def test_gemm_fp8_blockscaled(m, n, k):
    """Against fp32 matmul of the de-quantised operands: the only difference is summation order and
    the bf16 rounding of the output."""
    from rocshmem_b200.ops import gemm
    a_q, a_s, b_q, b_s, a_deq, b_deq = _fp8_inputs(m, n, k, seed=m + n)
    before = gemm.gemm_error_count()
    c = gemm.gemm_fp8_blockscaled(a_q, a_s, b_q, b_s)
    torch.cuda.synchronize()
    assert gemm.gemm_error_count() == before, "a GEMM CTA hit its wait budget"
    ok, err = close(c, a_deq @ b_deq.t(), k)
    assert ok, f"max abs error {err}"


def test_grouped_gemm_fp8_blockscaled():
    from rocshmem_b200.ops import gemm
    G, n, k = 5, 384, 1024
    sizes = [200, 0, 128, 77, 300]
    m = sum(sizes) + 9  # rows past offsets[-1] stay untouched
    a_q, a_s, b_q, b_s, a_deq, b_deq = _fp8_inputs(m, n, k, seed=3, groups=G)
    offsets = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32, device="cuda")
    out = torch.full((m, n), 7.0, dtype=torch.bfloat16, device="cuda")
    before = gemm.gemm_error_count()
    gemm.grouped_gemm_fp8_blockscaled(a_q, a_s, b_q, b_s, offsets, out=out)
    torch.cuda.synchronize()
    assert gemm.gemm_error_count() == before
    lo = 0
    for gi, sz in enumerate(sizes):
        if sz:
            ok, err = close(out[lo:lo + sz], a_deq[lo:lo + sz] @ b_deq[gi].t(), k)
            assert ok, (gi, err)
        lo += sz
    assert torch.all(out[lo:] == 7.0)


def test_grouped_gemm_fp8_swiglu():
    from rocshmem_b200.ops import gemm
    G, n, k = 3, 512, 1024   # 256 gate + 256 up rows per expert
    sizes = [130, 256, 40]
    m = sum(sizes)
    a_q, a_s, b_q, b_s, a_deq, b_deq = _fp8_inputs(m, n, k, seed=5, groups=G)
    offsets = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32, device="cuda")
    before = gemm.gemm_error_count()
    out = gemm.grouped_gemm_fp8_blockscaled(a_q, a_s, b_q, b_s, offsets, swiglu=True)
    torch.cuda.synchronize()
    assert gemm.gemm_error_count() == before
    assert out.shape == (m, n // 2)
    lo = 0
    for gi, sz in enumerate(sizes):
        hc = a_deq[lo:lo + sz] @ b_deq[gi].t()
        want = torch.nn.functional.silu(hc[:, :n // 2]) * hc[:, n // 2:]
        ok, err = close(out[lo:lo + sz], want, k)
        assert ok, (gi, err)
        lo += sz


@pytest.mark.parametrize("two_cta", [True, False])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (300, 520, 1024), (1000, 3584, 512), (129, 8, 256)])
def test_gemm_bf16_kernel_variants(m, n, k, two_cta):
    """The one-CTA and the two-CTA (cta_group::2) kernels, forced explicitly."""
    from rocshmem_b200.ops import gemm
    g = torch.Generator(device="cuda").manual_seed(m + k)
    a = (torch.randn(m, k, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(n, k, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    before = gemm.gemm_error_count()
    c = gemm.gemm_bf16(a, b, two_cta=two_cta)
    torch.cuda.synchronize()
    assert gemm.gemm_error_count() == before
    ok, err = close(c, ref_gemm(a, b), k)
    assert ok, f"max abs error {err}"


@pytest.mark.parametrize("swiglu", [False, True])
def test_grouped_gemm_with_gathered_rows(swiglu):
    """A rows picked by index inside the kernel (cp.async producer warps) against an fp32 matmul of the same rows
    gathered by PyTorch."""
    from rocshmem_b200.ops import gemm
    G, n, k, src_rows = 4, 512, 1024, 700
    sizes = [150, 0, 333, 129]
    total = sum(sizes)
    g = torch.Generator(device="cuda").manual_seed(17)
    src = (torch.randn(src_rows, k, generator=g, device="cuda") * 0.7).to(torch.bfloat16)
    b = (torch.randn(G, n, k, generator=g, device="cuda") * 0.3).to(torch.bfloat16)
    row_index = torch.randint(0, src_rows, (total + 40,), generator=g, device="cuda", dtype=torch.int32)
    offsets = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32, device="cuda")
    width = n // 2 if swiglu else n
    out = torch.full((total + 40, width), 7.0, dtype=torch.bfloat16, device="cuda")
    before = gemm.gemm_error_count()
    gemm.grouped_gemm_bf16_gathered(src, row_index, b, offsets, swiglu=swiglu, out=out)
    torch.cuda.synchronize()
    assert gemm.gemm_error_count() == before
    lo = 0
    for gi, sz in enumerate(sizes):
        if sz:
            hc = src.float()[row_index[lo:lo + sz].long()] @ b[gi].float().t()
            want = torch.nn.functional.silu(hc[:, :n // 2]) * hc[:, n // 2:] if swiglu else hc
            ok, err = close(out[lo:lo + sz], want, k)
            assert ok, (gi, err)
        lo += sz
    assert torch.all(out[lo:] == 7.0), "rows past offsets[-1] were written"


def test_block_scaled_moe_gemms_against_fp32():
    """The two block-scaled MoE GEMMs: gate/up with rows and scales gathered by index, SwiGLU and a quantising
    epilogue; down projection with the scatter-add epilogue."""
    from rocshmem_b200.ops import gemm, moe
    G, H, I, src_rows, dst_rows = 4, 1024, 512, 600, 600
    sizes = [140, 0, 260, 129]
    total = sum(sizes)
    g = torch.Generator(device="cuda").manual_seed(29)
    x = (torch.randn(src_rows, H, generator=g, device="cuda") * 0.7).to(torch.bfloat16)
    w13 = (torch.randn(G, 2 * I, H, generator=g, device="cuda") * H ** -0.5).to(torch.bfloat16)
    w2 = (torch.randn(G, H, I, generator=g, device="cuda") * I ** -0.5).to(torch.bfloat16)
    row_index = torch.randint(0, src_rows, (total,), generator=g, device="cuda", dtype=torch.int32)
    weights = torch.rand(total, generator=g, device="cuda")
    offsets = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32, device="cuda")
    xq, xs = moe.fp8_quantize_1x128(x)
    w13q, w13s = gemm.quantize_weight_128x128(w13)
    w2q, w2s = gemm.quantize_weight_128x128(w2)
    hq = torch.zeros(total + 8, I, dtype=torch.uint8, device="cuda")
    hs = torch.zeros(total + 8, I // 128, dtype=torch.float32, device="cuda")
    before = gemm.gemm_error_count()
    gemm.grouped_gemm_fp8_swiglu_quant(xq.view(torch.uint8), xs, w13q, w13s, offsets, hq, hs, row_index=row_index)
    torch.cuda.synchronize()
    assert gemm.gemm_error_count() == before
    x_ref = moe.ref_dequantize_1x128(xq, xs)
    w13_ref, w2_ref = gemm.dequantize_weight_128x128(w13q, w13s), gemm.dequantize_weight_128x128(w2q, w2s)
    h_got = moe.ref_dequantize_1x128(hq[:total].view(torch.float8_e4m3fn), hs[:total])
    lo = 0
    h_ref = torch.zeros(total, I, device="cuda")
    for gi, sz in enumerate(sizes):
        hc = x_ref[row_index[lo:lo + sz].long()] @ w13_ref[gi].t()
        h_ref[lo:lo + sz] = torch.nn.functional.silu(hc[:, :I]) * hc[:, I:]
        lo += sz
    # one e4m3 rounding step (2^-4 relative at the top of a block's range) on top of the GEMM's own error
    assert (h_got - h_ref).abs().max().item() <= 0.07 * h_ref.abs().max().item() + 1e-3
    assert torch.all(hq[total:] == 0), "rows past offsets[-1] were written"
    y = torch.zeros(dst_rows, H, dtype=torch.bfloat16, device="cuda")
    gemm.grouped_gemm_fp8_scatter_add(hq, hs, w2q, w2s, offsets, row_index, y, weights=weights)
    torch.cuda.synchronize()
    assert gemm.gemm_error_count() == before
    want = torch.zeros(dst_rows, H, device="cuda")
    lo = 0
    for gi, sz in enumerate(sizes):
        prod = (h_got[lo:lo + sz] @ w2_ref[gi].t()) * weights[lo:lo + sz].unsqueeze(1)
        want.index_add_(0, row_index[lo:lo + sz].long(), prod)
        lo += sz
    assert (y.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 0.05


@pytest.mark.parametrize("weighted", [False, True])
def test_grouped_gemm_scatter_add_epilogue(weighted):
    """y[row_index[p]] += w[p] * (a[p] @ b[g].T): several positions name the same destination row (the sum over a
    token's local experts), against an fp32 index_add of the per-position products."""
    from rocshmem_b200.ops import gemm
    G, n, k, dst_rows = 3, 1024, 512, 300
    sizes = [200, 131, 90]
    total = sum(sizes)
    g = torch.Generator(device="cuda").manual_seed(23)
    a = (torch.randn(total + 5, k, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(G, n, k, generator=g, device="cuda") * 0.3).to(torch.bfloat16)
    row_index = torch.randint(0, dst_rows, (total,), generator=g, device="cuda", dtype=torch.int32)
    w = torch.rand(total, generator=g, device="cuda") if weighted else None
    offsets = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32, device="cuda")
    y = torch.zeros((dst_rows, n), dtype=torch.bfloat16, device="cuda")
    before = gemm.gemm_error_count()
    gemm.grouped_gemm_bf16_scatter_add(a, b, offsets, row_index, y, weights=w)
    torch.cuda.synchronize()
    assert gemm.gemm_error_count() == before
    want = torch.zeros((dst_rows, n), dtype=torch.float32, device="cuda")
    lo = 0
    for gi, sz in enumerate(sizes):
        prod = a[lo:lo + sz].float() @ b[gi].float().t()
        if weighted:
            prod = prod * w[lo:lo + sz].unsqueeze(1)
        want.index_add_(0, row_index[lo:lo + sz].long(), prod.to(torch.bfloat16).float())
        lo += sz
    # Up to ~6 positions share a row; every partial sum is rounded to bf16 once more than in the reference.
    err = (y.float() - want).abs().max().item()
    assert err <= 2e-2 * want.abs().max().item() + 0.05, err
    untouched = torch.ones(dst_rows, dtype=torch.bool, device="cuda")
    untouched[row_index.long()] = False
    assert torch.all(y[untouched] == 0)


@pytest.mark.parametrize("kind", ["pair", "one_cta", "fp8", "grouped", "grouped_fp8"])
def test_headline_shapes_in_full(kind):
    """Every element of the tensor-parallel MLP and MoE expert shapes of the benchmarks against fp32 references."""
    from rocshmem_b200.ops import gemm, moe
    g = torch.Generator(device="cuda").manual_seed(101)
    before = gemm.gemm_error_count()
    if kind in ("pair", "one_cta", "fp8"):
        m, n, k = 8192, 3584, 8192
        a = (torch.randn(m, k, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
        b = (torch.randn(n, k, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
        if kind == "fp8":
            a_q, a_s = moe.fp8_quantize_1x128(a)
            b_q, b_s = gemm.quantize_weight_128x128(b)
            c = gemm.gemm_fp8_blockscaled(a_q, a_s, b_q, b_s)
            a_ref, b_ref = moe.ref_dequantize_1x128(a_q, a_s), gemm.dequantize_weight_128x128(b_q, b_s)
        else:
            c = gemm.gemm_bf16(a, b, two_cta=(kind == "pair"))
            a_ref, b_ref = a.float(), b.float()
        torch.cuda.synchronize()
        for lo in range(0, m, 2048):
            ok, err = close(c[lo:lo + 2048], a_ref[lo:lo + 2048] @ b_ref.t(), k)
            assert ok, (kind, lo, err)
    else:
        groups, n, k = 32, 4096, 7168           # 32 local experts, gate + up of intermediate 2048, hidden 7168
        sizes = torch.randint(900, 1150, (groups,), generator=g, device="cuda").tolist()
        rows = sum(sizes)
        offsets = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32, device="cuda")
        a = (torch.randn(rows, k, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
        b = (torch.randn(groups, n, k, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        if kind == "grouped_fp8":
            a_q, a_s = moe.fp8_quantize_1x128(a)
            b_q, b_s = gemm.quantize_weight_128x128(b)
            out = gemm.grouped_gemm_fp8_blockscaled(a_q, a_s, b_q, b_s, offsets, swiglu=True)
            a_ref, b_ref = moe.ref_dequantize_1x128(a_q, a_s), gemm.dequantize_weight_128x128(b_q, b_s)
        else:
            out = gemm.grouped_gemm_bf16(a, b, offsets, swiglu=True)
            a_ref, b_ref = a.float(), b.float()
        torch.cuda.synchronize()
        lo = 0
        for gi, sz in enumerate(sizes):
            hc = a_ref[lo:lo + sz] @ b_ref[gi].t()
            want = torch.nn.functional.silu(hc[:, :n // 2]) * hc[:, n // 2:]
            ok, err = close(out[lo:lo + sz], want, k)
            assert ok, (kind, gi, err)
            lo += sz
    assert gemm.gemm_error_count() == before

