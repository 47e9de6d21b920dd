"""tcgen05 / TMEM GEMMs (sm_100a) and the tensor-parallel kernels that fuse a GEMM with its collective.

All matrices are row-major bf16 and weights are given as ``[out_features, in_features]``, so every
operation computes ``A @ B.T`` with fp32 accumulation. The plain and grouped GEMMs work on ordinary
CUDA tensors; the fused tensor-parallel kernels work on symmetric-heap tensors, one PE per process.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import runtime as rt


def _stream(stream) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


def _check(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.bfloat16 or not t.is_contiguous() or not t.is_cuda:
        raise ValueError(f"{name} must be a contiguous bf16 CUDA tensor")
    if t.data_ptr() % 16:
        raise ValueError(f"{name} must be 16-byte aligned")


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None,
              two_cta: Optional[bool] = None) -> torch.Tensor:
    """``a [M, K] @ b [N, K].T -> [M, N]`` (bf16 in, fp32 accumulate in TMEM, bf16 out). By default the
    library picks the kernel (a pair of CTAs per 256 x 256 tile, ``tcgen05`` ``cta_group::2``, when M > 128);
    ``two_cta`` forces one or the other."""
    _check(a, "a")
    _check(b, "b")
    M, K = a.shape
    N, K2 = b.shape
    if K != K2 or K % 8:
        raise ValueError("inner dimensions must match and be a multiple of 8")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    else:
        _check(out, "out")
        if tuple(out.shape) != (M, N):
            raise ValueError(f"out must be [{M}, {N}]")
    C = rt._C()
    fn = C.gemm_bf16 if two_cta is None else (C.gemm_bf16_pair if two_cta else C.gemm_bf16_one_cta)
    fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, _stream(stream))
    return out


def grouped_gemm_bf16(a: torch.Tensor, b: torch.Tensor, offsets: torch.Tensor, swiglu: bool = False,
                      out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """Rows ``offsets[g]:offsets[g+1]`` of ``a [rows, K]`` are multiplied with ``b[g] [N, K]``.

    ``offsets`` is an int32 device tensor of ``groups + 1`` entries (its values are read on the GPU, so
    no host synchronisation is needed when they come out of the MoE dispatch). With ``swiglu`` the
    weight holds the gate projection in rows ``[0, N/2)`` and the up projection in ``[N/2, N)`` and the
    result is ``silu(gate) * up`` of width ``N / 2``. Rows past ``offsets[-1]`` are left untouched.
    """
    _check(a, "a")
    _check(b, "b")
    rows, K = a.shape
    G, N, K2 = b.shape
    if K != K2 or offsets.dtype != torch.int32 or offsets.numel() != G + 1:
        raise ValueError("grouped_gemm_bf16: shape mismatch")
    width = N // 2 if swiglu else N
    if out is None:
        out = torch.empty((rows, width), dtype=torch.bfloat16, device=a.device)
    rt._C().grouped_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), offsets.data_ptr(), G, rows, N, K,
                              int(swiglu), _stream(stream))
    return out


def grouped_gemm_bf16_gathered(a_rows: torch.Tensor, row_index: torch.Tensor, b: torch.Tensor, offsets: torch.Tensor,
                               swiglu: bool = False, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """:func:`grouped_gemm_bf16` whose A rows are gathered inside the kernel: position ``p`` of the grouped order
    reads row ``row_index[p]`` of ``a_rows [*, K]`` (bf16). ``out`` must hold at least ``offsets[-1]`` rows (its row
    count bounds nothing on the device)."""
    _check(a_rows, "a_rows")
    _check(b, "b")
    K = a_rows.shape[1]
    G, N, K2 = b.shape
    if K != K2 or K % 64 or offsets.dtype != torch.int32 or offsets.numel() != G + 1 or row_index.dtype != torch.int32:
        raise ValueError("grouped_gemm_bf16_gathered: shape mismatch (K must be a multiple of 64)")
    width = N // 2 if swiglu else N
    if out is None:
        out = torch.empty((row_index.numel(), width), dtype=torch.bfloat16, device=a_rows.device)
    rt._C().grouped_gemm_bf16_gathered(a_rows.data_ptr(), row_index.data_ptr(), b.data_ptr(), out.data_ptr(),
                                       offsets.data_ptr(), G, N, K, int(swiglu), _stream(stream))
    return out


def grouped_gemm_bf16_scatter_add(a: torch.Tensor, b: torch.Tensor, offsets: torch.Tensor, row_index: torch.Tensor,
                                  y: torch.Tensor, weights: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """``y[row_index[p]] += weights[p] * (a[p] @ b[g].T)`` for every position ``p`` of group ``g``: the grouped GEMM
    with the per-row weighted sum fused into its epilogue. ``y [*, N]`` bf16 must hold zeros (or the values to add
    to); several positions may name the same row."""
    _check(a, "a")
    _check(b, "b")
    _check(y, "y")
    rows, K = a.shape
    G, N, K2 = b.shape
    if K != K2 or y.shape[1] != N or N % 8 or offsets.numel() != G + 1 or row_index.dtype != torch.int32:
        raise ValueError("grouped_gemm_bf16_scatter_add: shape mismatch")
    if weights is not None and (weights.dtype != torch.float32 or not weights.is_contiguous()):
        raise ValueError("grouped_gemm_bf16_scatter_add: weights must be contiguous fp32")
    rt._C().grouped_gemm_bf16_scatter_add(a.data_ptr(), b.data_ptr(), y.data_ptr(), offsets.data_ptr(),
                                          row_index.data_ptr(), weights.data_ptr() if weights is not None else 0, G,
                                          rows, N, K, _stream(stream))
    return y


def grouped_gemm_fp8_swiglu_quant(a_q: torch.Tensor, a_scale: torch.Tensor, b_q: torch.Tensor, b_scale: torch.Tensor,
                                  offsets: torch.Tensor, out_q: torch.Tensor, out_s: torch.Tensor,
                                  row_index: Optional[torch.Tensor] = None, stream=None):
    """Block-scaled gate/up projection with SwiGLU whose result leaves the kernel as the next GEMM's operand:
    ``out_q [rows, N / 2]`` e4m3 with one fp32 scale per 128 columns in ``out_s [rows, N / 256]``. With
    ``row_index`` the A rows (``a_q [*, K]`` e4m3, ``a_scale [*, K / 128]``) are gathered inside the kernel:
    position ``p`` of the grouped order reads row ``row_index[p]``."""
    K = a_q.shape[1]
    G, N, K2 = b_q.shape
    if K != K2 or K % 512 or N % 256 or offsets.numel() != G + 1 or out_q.shape[1] != N // 2:
        raise ValueError("grouped_gemm_fp8_swiglu_quant: shape mismatch (K % 512, N % 256)")
    if tuple(a_scale.shape) != (a_q.shape[0], K // 128) or tuple(out_s.shape) != (out_q.shape[0], N // 256):
        raise ValueError("grouped_gemm_fp8_swiglu_quant: scale shapes")
    for t in (a_q, a_scale, b_q, b_scale, out_q, out_s):
        if not t.is_contiguous():
            raise ValueError("grouped_gemm_fp8_swiglu_quant: tensors must be contiguous")
    rt._C().grouped_gemm_fp8_swiglu_quant(a_q.data_ptr(), a_scale.data_ptr(),
                                          row_index.data_ptr() if row_index is not None else 0, b_q.data_ptr(),
                                          b_scale.data_ptr(), out_q.data_ptr(), out_s.data_ptr(), offsets.data_ptr(), G,
                                          a_q.shape[0], N, K, _stream(stream))
    return out_q, out_s


def grouped_gemm_fp8_scatter_add(a_q: torch.Tensor, a_scale: torch.Tensor, b_q: torch.Tensor, b_scale: torch.Tensor,
                                 offsets: torch.Tensor, row_index: torch.Tensor, y: torch.Tensor,
                                 weights: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """Block-scaled form of :func:`grouped_gemm_bf16_scatter_add`."""
    rows, K = a_q.shape
    G, N, K2 = b_q.shape
    if K != K2 or K % 512 or N % 128 or y.shape[1] != N or offsets.numel() != G + 1:
        raise ValueError("grouped_gemm_fp8_scatter_add: shape mismatch (K % 512, N % 128)")
    rt._C().grouped_gemm_fp8_scatter_add(a_q.data_ptr(), a_scale.data_ptr(), b_q.data_ptr(), b_scale.data_ptr(),
                                         y.data_ptr(), offsets.data_ptr(), row_index.data_ptr(),
                                         weights.data_ptr() if weights is not None else 0, G, rows, N, K,
                                         _stream(stream))
    return y


def gemm_error_count() -> int:
    """Number of GEMM CTAs (since process start) whose bounded wait expired; 0 in a healthy run."""
    return rt._C().gemm_error_count()


def _free_buffer_tables(*tables) -> None:
    """Collective: free every symmetric tensor held in the per-shape buffer tables, then clear them."""
    tensors = [v for table in tables for entry in table.values() for v in entry if isinstance(v, torch.Tensor)]
    if tensors and rt.is_cuda():
        torch.cuda.synchronize()
    rt.free_all(tensors)
    for table in tables:
        table.clear()


class TensorParallelLinear:
    """Buffers and calls of the fused tensor-parallel kernels for one (m_shard, K, N) shape.

    * :meth:`ag_gemm`: ``concat_ranks(x_shard) @ w.T`` where every rank contributes ``x_shard
      [m_shard, K]`` (all-gather fused into the GEMM's A-operand pipeline);
    * :meth:`gemm_rs`: ``reduce_scatter_ranks(a @ w.T)`` where ``a [n_ranks * m_shard, K_local]`` and
      the rank keeps rows ``[rank * m_shard, (rank + 1) * m_shard)`` of the sum.
    """

    def __init__(self, m_shard: int, team: Optional[rt.Team] = None):
        if rt.n_local_pes() != 1:
            raise RuntimeError("the fused tensor-parallel kernels need one PE per process")
        self.team = team or rt.team_world()
        self.n_ranks = self.team.n_pes()
        self.m_shard = m_shard
        self._ag = {}
        self._rs = {}
        self.kernel_launches = 0

    def destroy(self) -> None:
        """Collective: give the gather, staging and flag buffers of every shape used so far back to the heap."""
        _free_buffer_tables(self._ag, self._rs)

    def ag_input(self, k: int) -> torch.Tensor:
        """The symmetric ``[m_shard, k]`` buffer that holds this rank's activation shard."""
        return self._ag_buffers(k)[0]

    def _ag_buffers(self, k: int):
        if k not in self._ag:
            x = rt.zeros((self.m_shard, k), torch.bfloat16)
            gathered = rt.zeros((self.n_ranks * self.m_shard, k), torch.bfloat16)
            flags = rt.zeros(max(16, self.n_ranks * self.m_shard // 128), torch.int64)
            self._ag[k] = [x, gathered, flags, 0]
        return self._ag[k]

    def ag_gemm(self, w: torch.Tensor, out: Optional[torch.Tensor] = None, swiglu: bool = False,
                stream=None) -> torch.Tensor:
        """Uses the current content of :meth:`ag_input` on every rank. ``w [N, K]`` local weight shard.

        With ``swiglu`` the weight holds gate rows ``[0, N/2)`` and up rows ``[N/2, N)`` and the result
        is ``silu(gate) * up`` of width ``N / 2`` (the activation is applied in the GEMM epilogue)."""
        _check(w, "w")
        N, K = w.shape
        buf = self._ag_buffers(K)
        x, gathered, flags = buf[0], buf[1], buf[2]
        buf[3] += 1
        if out is None:
            out = torch.empty((self.n_ranks * self.m_shard, N // 2 if swiglu else N), dtype=torch.bfloat16,
                              device=w.device)
        rt._C().ag_gemm_bf16(self.team.handle, x.data_ptr(), gathered.data_ptr(), flags.data_ptr(), w.data_ptr(),
                             out.data_ptr(), self.m_shard, N, K, buf[3], int(swiglu), _stream(stream))
        self.kernel_launches += 1
        return out

    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        """``a [n_ranks * m_shard, K_local]``, ``w [N, K_local]`` -> this rank's ``[m_shard, N]`` rows of the
        sum over ranks of ``a @ w.T``."""
        _check(a, "a")
        _check(w, "w")
        N, K = w.shape
        if a.shape[0] != self.n_ranks * self.m_shard or a.shape[1] != K:
            raise ValueError("gemm_rs: a must be [n_ranks * m_shard, K_local]")
        if N not in self._rs:
            # staging slices of every rank's partial of my rows, and the grid counter's 128 bytes
            self._rs[N] = [rt.zeros((self.n_ranks, self.m_shard, N), torch.bfloat16), rt.zeros(16, torch.int64), 0]
        entry = self._rs[N]
        staging, counter = entry[0], entry[1]
        entry[2] += 1
        if out is None:
            out = torch.empty((self.m_shard, N), dtype=torch.bfloat16, device=a.device)
        rt._C().gemm_rs_bf16(self.team.handle, a.data_ptr(), w.data_ptr(), staging.data_ptr(), out.data_ptr(),
                             self.m_shard, N, K, counter.data_ptr(), entry[2], _stream(stream))
        self.kernel_launches += 1
        return out


# ---- block-scaled fp8 ---------------------------------------------------------------------------------------------

E4M3_MAX = 448.0


def quantize_weight_128x128(w: torch.Tensor):
    """``w [..., N, K]`` (N, K multiples of 128) -> (e4m3 ``[..., N, K]``, fp32 scales ``[..., N/128, K/128]``)
    with one scale per 128 x 128 block (``w ~ q * scale``). Plain PyTorch: weights are quantised once."""
    *lead, N, K = w.shape
    blocks = w.float().reshape(*lead, N // 128, 128, K // 128, 128)
    amax = blocks.abs().amax(dim=(-3, -1), keepdim=True)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (blocks / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).reshape(*lead, N, K)
    return q.contiguous(), scale.reshape(*lead, N // 128, K // 128).contiguous()


def dequantize_weight_128x128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """fp32 weight from e4m3 values and one scale per 128 x 128 block (reference for tests)."""
    *lead, N, K = q.shape
    blocks = q.float().reshape(*lead, N // 128, 128, K // 128, 128)
    return (blocks * scale.reshape(*lead, N // 128, 1, K // 128, 1)).reshape(*lead, N, K)


def _check8(q: torch.Tensor, s: torch.Tensor, name: str) -> None:
    if q.dtype not in (torch.float8_e4m3fn, torch.uint8) or not q.is_contiguous() or not q.is_cuda:
        raise ValueError(f"{name} must be a contiguous e4m3 CUDA tensor")
    if s.dtype != torch.float32 or not s.is_contiguous() or s.data_ptr() % 16 or q.data_ptr() % 16:
        raise ValueError(f"{name} scales must be contiguous fp32, 16-byte aligned")


def gemm_fp8_blockscaled(a_q: torch.Tensor, a_scale: torch.Tensor, b_q: torch.Tensor, b_scale: torch.Tensor,
                         out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """``(a_q * a_scale) [M, K] @ (b_q * b_scale) [N, K].T -> [M, N]`` bf16. ``a_scale [M, K/128]`` (1 x 128
    blocks, as produced by :func:`rocshmem_b200.ops.moe.fp8_quantize_1x128` and by the MoE dispatch),
    ``b_scale [N/128, K/128]`` (128 x 128 blocks). K a multiple of 512, N of 128."""
    _check8(a_q, a_scale, "a")
    _check8(b_q, b_scale, "b")
    M, K = a_q.shape
    N, K2 = b_q.shape
    if K != K2 or K % 512 or N % 128 or tuple(a_scale.shape) != (M, K // 128) or tuple(b_scale.shape) != (N // 128, K // 128):
        raise ValueError("gemm_fp8_blockscaled: shape mismatch (K % 512 == 0, N % 128 == 0)")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a_q.device)
    rt._C().gemm_fp8_blockscaled(a_q.data_ptr(), a_scale.data_ptr(), b_q.data_ptr(), b_scale.data_ptr(),
                                 out.data_ptr(), M, N, K, _stream(stream))
    return out


def grouped_gemm_fp8_blockscaled(a_q: torch.Tensor, a_scale: torch.Tensor, b_q: torch.Tensor, b_scale: torch.Tensor,
                                 offsets: torch.Tensor, swiglu: bool = False, out: Optional[torch.Tensor] = None,
                                 stream=None) -> torch.Tensor:
    """Grouped form: rows ``offsets[g]:offsets[g+1]`` of ``a_q [rows, K]`` use ``b_q[g] [N, K]`` with
    ``b_scale[g] [N/128, K/128]``; ``offsets`` int32 on the device. With ``swiglu`` (N a multiple of
    256, gate rows first) the result is ``silu(gate) * up`` of width ``N / 2``."""
    _check8(a_q, a_scale, "a")
    _check8(b_q, b_scale, "b")
    rows, K = a_q.shape
    G, N, K2 = b_q.shape
    if K != K2 or K % 512 or N % 128 or offsets.dtype != torch.int32 or offsets.numel() != G + 1:
        raise ValueError("grouped_gemm_fp8_blockscaled: shape mismatch")
    if out is None:
        out = torch.empty((rows, N // 2 if swiglu else N), dtype=torch.bfloat16, device=a_q.device)
    rt._C().grouped_gemm_fp8_blockscaled(a_q.data_ptr(), a_scale.data_ptr(), b_q.data_ptr(), b_scale.data_ptr(),
                                         out.data_ptr(), offsets.data_ptr(), G, rows, N, K, int(swiglu),
                                         _stream(stream))
    return out


def quantize_1x128_into(x: torch.Tensor, q: torch.Tensor, scales: torch.Tensor, stream=None) -> None:
    """1 x 128 block-scaled e4m3 quantisation of ``x [rows, hidden]`` bf16 into caller-provided ``q``
    (e4m3 / uint8, same shape) and ``scales [rows, hidden / 128]`` fp32 (e.g. symmetric-heap buffers)."""
    rows, hidden = x.shape
    rt._C().fp8_quantize_1x128(x.data_ptr(), q.data_ptr(), scales.data_ptr(), rows, hidden, _stream(stream))


class TensorParallelLinearFp8:
    """Block-scaled e4m3 versions of the fused tensor-parallel kernels (see :class:`TensorParallelLinear`).

    Activations carry 1 x 128 scales and travel over NVLink as e4m3 (half the bytes of bf16); weights carry
    128 x 128 scales (:func:`quantize_weight_128x128`). Outputs are bf16."""

    def __init__(self, m_shard: int, team: Optional[rt.Team] = None):
        if rt.n_local_pes() != 1:
            raise RuntimeError("the fused tensor-parallel kernels need one PE per process")
        self.team = team or rt.team_world()
        self.n_ranks = self.team.n_pes()
        self.m_shard = m_shard
        self._ag = {}
        self._rs = {}
        self.kernel_launches = 0

    def destroy(self) -> None:
        """Collective: give the gather, staging and flag buffers of every shape used so far back to the heap."""
        _free_buffer_tables(self._ag, self._rs)

    def _ag_buffers(self, k: int):
        if k not in self._ag:
            M = self.n_ranks * self.m_shard
            self._ag[k] = [rt.zeros((self.m_shard, k), torch.uint8), rt.zeros((self.m_shard, k // 128), torch.float32),
                           rt.zeros((M, k), torch.uint8), rt.zeros((M, k // 128), torch.float32),
                           rt.zeros(max(16, M // 128), torch.int64), 0]
        return self._ag[k]

    def ag_input(self, k: int):
        """The symmetric ``(e4m3 [m_shard, k] as uint8, scales [m_shard, k / 128])`` pair that holds this
        rank's quantised activation shard."""
        buf = self._ag_buffers(k)
        return buf[0], buf[1]

    def set_input(self, x_shard: torch.Tensor, stream=None) -> None:
        """Quantises ``x_shard [m_shard, k]`` bf16 straight into :meth:`ag_input`."""
        q, s = self.ag_input(x_shard.shape[1])
        quantize_1x128_into(x_shard, q, s, stream)
        self.kernel_launches += 1

    def ag_gemm(self, w_q: torch.Tensor, w_s: torch.Tensor, out: Optional[torch.Tensor] = None, swiglu: bool = False,
                stream=None) -> torch.Tensor:
        """All-gather of the quantised activations fused with ``gathered @ w.T`` (block-scaled e4m3), optionally with SwiGLU."""
        N, K = w_q.shape
        x_q, x_s, g_q, g_s, flags, _ = buf = self._ag_buffers(K)
        buf[5] += 1
        if out is None:
            out = torch.empty((self.n_ranks * self.m_shard, N // 2 if swiglu else N), dtype=torch.bfloat16,
                              device=w_q.device)
        rt._C().ag_gemm_fp8(self.team.handle, x_q.data_ptr(), x_s.data_ptr(), g_q.data_ptr(), g_s.data_ptr(),
                            flags.data_ptr(), w_q.data_ptr(), w_s.data_ptr(), out.data_ptr(), self.m_shard, N, K,
                            buf[5], int(swiglu), _stream(stream))
        self.kernel_launches += 1
        return out

    def gemm_rs(self, a_q: torch.Tensor, a_s: torch.Tensor, w_q: torch.Tensor, w_s: torch.Tensor,
                out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        """``a @ w.T`` (block-scaled e4m3) fused with the reduce-scatter of the bf16 result over the team."""
        N, K = w_q.shape
        if a_q.shape[0] != self.n_ranks * self.m_shard or a_q.shape[1] != K:
            raise ValueError("gemm_rs: a must be [n_ranks * m_shard, K_local]")
        if N not in self._rs:
            # staging slices of every rank's partial of my rows, and the grid counter's 128 bytes
            self._rs[N] = [rt.zeros((self.n_ranks, self.m_shard, N), torch.bfloat16), rt.zeros(16, torch.int64), 0]
        entry = self._rs[N]
        entry[2] += 1
        if out is None:
            out = torch.empty((self.m_shard, N), dtype=torch.bfloat16, device=a_q.device)
        rt._C().gemm_rs_fp8(self.team.handle, a_q.data_ptr(), a_s.data_ptr(), w_q.data_ptr(), w_s.data_ptr(),
                            entry[0].data_ptr(), out.data_ptr(), self.m_shard, N, K, entry[1].data_ptr(), entry[2],
                            _stream(stream))
        self.kernel_launches += 1
        return out
