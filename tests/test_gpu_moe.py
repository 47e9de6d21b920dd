"""MoE expert-parallel dispatch / combine and the block-scaled fp8 helpers against plain PyTorch fp32
references. Several PEs share the one GPU (one cooperative launch per operation)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

NPES = 4


@pytest.fixture(scope="module")
def shm():
    import rocshmem_b200 as s
    if s.is_initialized():
        s.finalize()
    s.init(n_local=NPES, heap_size="1G", ROCSHMEM_WAIT_TIMEOUT_MS=5000)
    yield s
    torch.cuda.synchronize()
    s.finalize()


def check_clean(shm):
    torch.cuda.synchronize()
    for l in range(NPES):
        err = shm.get_error(l)
        assert err["count"] == 0, err


def make_inputs(shm, T, H, E, K, seed, drop_some=False):
    from rocshmem_b200.ops import moe
    dev = shm.device()
    x = shm.zeros((T, H), torch.bfloat16)
    idx = shm.zeros((T, K), torch.int32)
    w = shm.zeros((T, K), torch.float32)
    host = []
    for l in range(NPES):
        g = torch.Generator().manual_seed(seed * 100 + l)
        xl = torch.randn(T, H, generator=g).to(torch.bfloat16)
        il, wl = moe.make_routing(T, E, K, seed * 1000 + l)
        if drop_some:
            il[::5, -1] = -1  # unused top-k entries
            il[3] = -1        # a token that goes nowhere
        shm.local_view(x, l).copy_(xl.to(dev))
        shm.local_view(idx, l).copy_(il.to(dev))
        shm.local_view(w, l).copy_(wl.to(dev))
        host.append((xl, il, wl))
    torch.cuda.synchronize()
    return x, idx, w, host


def check_expert_pairs(shm, d, res, K, epr):
    """The pair lists written by the dispatch kernel against a brute-force grouping of the metadata."""
    offsets, lay_row, lay_k, lay_w = d.expert_pairs()
    for l in range(NPES):
        off = shm.local_view(offsets, l).cpu().tolist()
        rows = shm.local_view(lay_row, l).cpu()
        ks = shm.local_view(lay_k, l).cpu()
        ws = shm.local_view(lay_w, l).cpu()
        meta = shm.local_view(res.recv_meta, l).cpu()
        info = shm.local_view(res.recv_info, l).cpu().tolist()
        live = [r for s in range(NPES) for r in range(info[1 + s], info[1 + s] + info[1 + NPES + s])]
        assert off[0] == 0 and off[-1] == sum(int((meta[r, 0:K] >= 0).sum()) for r in live)
        for e in range(epr):
            got = sorted(zip(rows[off[e]:off[e + 1]].tolist(), ks[off[e]:off[e + 1]].tolist()))
            want = sorted((r, k) for r in live for k in range(K) if meta[r, k] == e)
            assert got == want, (l, e)
            for p in range(off[e], off[e + 1]):
                assert ws[p].item() == meta[rows[p], 8 + ks[p]].view(torch.float32).item()


@pytest.mark.parametrize("mode", ["fixed-compact", "fixed-slotted", "staged-compact", "staged-slotted", "low-latency"])
@pytest.mark.parametrize("T,H,E,K", [(96, 1024, 16, 4), (257, 7168, 32, 8), (8, 512, 4, 2)])
def test_dispatch_fp8_and_combine(shm, mode, T, H, E, K):
    from rocshmem_b200.ops import moe
    low_latency = mode == "low-latency"
    layout = "slotted" if low_latency else mode.split("-")[1]
    d = moe.EpDispatcher(E, K, H, T + 3, layout=layout, dynamic=mode.startswith("staged"), low_latency=low_latency,
                         expert_layout=True)
    epr = E // NPES
    for rep in range(3):  # repeated use exercises the epoch / double-buffer logic
        x, idx, w, host = make_inputs(shm, T, H, E, K, seed=rep + 1, drop_some=(rep == 1))
        res = d.dispatch(x, idx, w)
        check_clean(shm)
        ref_rows = moe.ref_dispatch([h[1] for h in host], NPES, E)
        for dst in range(NPES):
            info = shm.local_view(res.recv_info, dst).cpu().tolist()
            want = ref_rows[dst]
            assert info[0] == len(want), (dst, info[0], len(want))
            meta = shm.local_view(res.recv_meta, dst).cpu()
            qx = shm.local_view(res.recv_x.view(torch.uint8), dst).view(torch.float8_e4m3fn).cpu()
            sc = shm.local_view(res.recv_scales, dst).cpu()
            pairs_per_expert = [0] * epr
            pos = 0
            for s in range(NPES):
                first, count = info[1 + s], info[1 + NPES + s]
                src_list = [(ss, t) for ss, t in want if ss == s]
                assert count == len(src_list)
                assert first == (s * (T + 3) if layout == "slotted" else pos)
                pos += count
                if count == 0:
                    continue
                rows = slice(first, first + count)
                if low_latency:
                    # Rows of one source arrive in the order its blocks took their slots: sort by token.
                    rows = first + torch.argsort(meta[rows, 16])
                assert meta[rows, 16].tolist() == [t for _, t in src_list]
                assert meta[rows, 17].tolist() == [s] * count
                xs, is_, ws = host[s]
                toks = torch.tensor([t for _, t in src_list])
                q_ref, s_ref = moe.ref_quantize_1x128(xs[toks])
                assert torch.allclose(sc[rows], s_ref, rtol=1e-6, atol=0)
                got = moe.ref_dequantize_1x128(qx[rows], sc[rows])
                ref = moe.ref_dequantize_1x128(q_ref, s_ref)
                # identical scales; allow one e4m3 rounding step of difference at ties
                assert (got - ref).abs().max() <= 0.075 * xs[toks].float().abs().max()
                assert (got - xs[toks].float()).abs().max() <= 0.075 * xs[toks].float().abs().max() + 1e-3
                gi = is_[toks]
                local = torch.where((gi >= 0) & (gi // epr == dst), gi % epr, torch.full_like(gi, -1))
                assert torch.equal(meta[rows, 0:K], local)
                assert torch.equal(meta[rows, 8:8 + K].view(torch.float32), ws[toks])
                for e in local.flatten().tolist():
                    if e >= 0:
                        pairs_per_expert[e] += 1
            assert info[1 + 2 * NPES:1 + 2 * NPES + epr] == pairs_per_expert
        check_expert_pairs(shm, d, res, K, epr)
        # combine with "identity experts": y = dequantised input, weighted sum returns the token
        y = d.result_buffer()
        for l in range(NPES):
            q = shm.local_view(res.recv_x.view(torch.uint8), l).view(torch.float8_e4m3fn)
            deq = moe.ref_dequantize_1x128(q, shm.local_view(res.recv_scales, l))
            shm.local_view(y, l).copy_(deq.to(torch.bfloat16))
        out = shm.zeros((T, H), torch.bfloat16)
        d.combine(y, idx, w, T, weighted=True, out=out)
        check_clean(shm)
        for l in range(NPES):
            xs, is_, ws = host[l]
            got = shm.local_view(out, l).float().cpu()
            wsum = torch.where(is_ >= 0, ws, torch.zeros_like(ws)).sum(-1, keepdim=True)
            want = xs.float() * wsum
            assert (got - want).abs().max() <= 0.08 * xs.float().abs().max() + 2e-2
        # unweighted combine of rank-constant rows is exact: sum of (rank + 1) over the token's ranks
        for l in range(NPES):
            shm.local_view(y, l).fill_(float(l + 1))
        d.combine(y, idx, w, T, weighted=False, out=out)
        check_clean(shm)
        for l in range(NPES):
            is_ = host[l][1]
            want = torch.zeros(T)
            for t in range(T):
                ranks = set(int(e) // epr for e in is_[t].tolist() if e >= 0)
                want[t] = sum(r + 1 for r in ranks)
            got = shm.local_view(out, l).float().cpu()
            assert torch.equal(got[:, 0], want) and torch.equal(got[:, -1], want)
        for t in (out, w, idx, x):
            shm.free(t)
    d.destroy()


@pytest.mark.parametrize("dynamic", [False, True])
def test_dispatch_bf16_rows_are_exact(shm, dynamic):
    from rocshmem_b200.ops import moe
    T, H, E, K = 130, 2048, 8, 3
    d = moe.EpDispatcher(E, K, H, T, quantize=False, dynamic=dynamic)
    x, idx, w, host = make_inputs(shm, T, H, E, K, seed=9)
    res = d.dispatch(x, idx, w)
    check_clean(shm)
    ref_rows = moe.ref_dispatch([h[1] for h in host], NPES, E)
    for dst in range(NPES):
        rows = shm.local_view(res.recv_x, dst).cpu()
        want = torch.stack([host[s][0][t] for s, t in ref_rows[dst]])
        assert torch.equal(rows[:len(ref_rows[dst])], want)


def test_expert_layout_lists(shm):
    from rocshmem_b200.ops import moe
    T, H, E, K = 200, 512, 16, 4
    d = moe.EpDispatcher(E, K, H, T)
    x, idx, w, host = make_inputs(shm, T, H, E, K, seed=4)
    res = d.dispatch(x, idx, w)
    offsets, row_index, pair_k = d.expert_layout()
    check_clean(shm)
    epr = E // NPES
    for l in range(NPES):
        off = shm.local_view(offsets, l).cpu().tolist()
        rows = shm.local_view(row_index, l).cpu()
        ks = shm.local_view(pair_k, l).cpu()
        meta = shm.local_view(res.recv_meta, l).cpu()
        n = shm.local_view(res.recv_info, l).cpu()[0].item()
        assert off[0] == 0 and off[-1] == int((meta[:n, 0:K] >= 0).sum())
        for e in range(epr):
            got = sorted(zip(rows[off[e]:off[e + 1]].tolist(), ks[off[e]:off[e + 1]].tolist()))
            want = sorted((r, k) for r in range(n) for k in range(K) if meta[r, k] == e)
            assert got == want


@pytest.mark.parametrize("rows,hidden", [(1, 512), (33, 7168), (1000, 1024)])
def test_fp8_quantize_dequantize(shm, rows, hidden):
    from rocshmem_b200.ops import moe
    g = torch.Generator().manual_seed(rows)
    x = (torch.randn(rows, hidden, generator=g) * 3).to(torch.bfloat16)
    x[0, :128] = 0  # an all-zero block keeps scale 1 and zeros
    xd = x.cuda()
    q, s = moe.fp8_quantize_1x128(xd)
    q_ref, s_ref = moe.ref_quantize_1x128(x)
    assert torch.allclose(s.cpu(), s_ref, rtol=1e-6, atol=0)
    deq = moe.fp8_dequantize_1x128(q, s).float().cpu()
    ref = moe.ref_dequantize_1x128(q_ref, s_ref)
    # one e4m3 step at the top of a block's range is amax * 32 / 448
    assert (deq - ref).abs().max() <= 0.075 * x.float().abs().max()
    assert (deq - x.float()).abs().max() <= 0.075 * x.float().abs().max()
    assert torch.all(deq[0, :128] == 0)
    # most elements must agree bit for bit with the reference rounding
    same = (q.cpu().view(torch.uint8) == q_ref.view(torch.uint8)).float().mean().item()
    assert same > 0.999, same
