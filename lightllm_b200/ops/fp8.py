"""fp8 (e4m3) weights with 128 x 128 block scales and per-token-group activation scales: the DeepSeek-V3
checkpoint scheme (`weight` e4m3 + `weight_scale_inv` [N/128, K/128] fp32).

Reference behaviour: lightllm/common/quantization/deepgemm.py:46-126 (method `fp8w8a8-b128-deepgemm`: activations
are quantised per token and 128-wide K group, then `deep_gemm.fp8_gemm_nt`), lightllm/common/quantization/w8a8.py
(the vllm / triton variants of the same scheme).  Here the GEMM is `csrc/gemm_fp8.cu` (tcgen05 kind::f8f6f4 with
the scales applied per K group on the way out of tensor memory); on CPU the same arithmetic runs in fp32.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _count
from ._native import check, i64, kernels, ptr, stream

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
GROUP = 128
EPI = {"store": 0, "residual": 1, "gated_silu": 2}


def _cdiv(a, b):
    return (a + b - 1) // b


def quant_weight_block(w: torch.Tensor, rows: int = GROUP):
    """[N, K] float -> (e4m3 [N, K], scale [ceil(N/rows), ceil(K/128)] fp32), one scale per rows x 128 block."""
    N, K = w.shape
    nb, kb = _cdiv(N, rows), _cdiv(K, GROUP)
    wp = torch.zeros(nb * rows, kb * GROUP, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    blocks = wp.view(nb, rows, kb, GROUP)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-10)
    scale = amax / FP8_MAX
    q = (blocks / scale.view(nb, 1, kb, 1)).clamp(-FP8_MAX, FP8_MAX).view(nb * rows, kb * GROUP)[:N, :K]
    return q.to(FP8).contiguous(), scale.contiguous()


def quant_act_reference(x: torch.Tensor):
    """[M, K] -> (e4m3 [M, K], scale [ceil(K/128), M] fp32): per token and 128-wide K group."""
    M, K = x.shape
    kb = _cdiv(K, GROUP)
    xp = torch.zeros(M, kb * GROUP, dtype=torch.float32, device=x.device)
    xp[:, :K] = x.float()
    g = xp.view(M, kb, GROUP)
    scale = g.abs().amax(dim=2).clamp_min(1e-10) / FP8_MAX
    q = (g / scale.unsqueeze(2)).clamp(-FP8_MAX, FP8_MAX).view(M, kb * GROUP)[:, :K]
    return q.to(FP8).contiguous(), scale.t().contiguous()


def dequant_act(xq: torch.Tensor, xs: torch.Tensor) -> torch.Tensor:
    M, K = xq.shape
    s = xs.t()[:M].repeat_interleave(GROUP, dim=1)[:, :K]
    return xq.float() * s


class Fp8Weight:
    """A [N, K] e4m3 weight with one fp32 scale per `ws_rows` x 128 block (ws_rows = 128: checkpoint layout;
    32: gate / up matrices interleaved in 32-row blocks for the gated epilogue).  For stacked expert weights
    [E * N, K] every expert's N must be a multiple of ws_rows."""

    def __init__(self, q: torch.Tensor, scale: torch.Tensor, ws_rows: int = GROUP):
        assert q.dtype == FP8 and q.dim() == 2 and scale.dtype == torch.float32
        assert scale.shape == (_cdiv(q.shape[0], ws_rows), _cdiv(q.shape[1], GROUP)), (q.shape, scale.shape, ws_rows)
        self.q, self.scale, self.ws_rows = q.contiguous(), scale.contiguous(), ws_rows
        self.shape = tuple(q.shape)
        self.device, self.dtype = q.device, torch.bfloat16

    @classmethod
    def from_float(cls, w: torch.Tensor, ws_rows: int = GROUP) -> "Fp8Weight":
        q, s = quant_weight_block(w, ws_rows)
        return cls(q, s, ws_rows)

    def to(self, device) -> "Fp8Weight":
        return Fp8Weight(self.q.to(device), self.scale.to(device), self.ws_rows)

    def dequant(self) -> torch.Tensor:
        N, K = self.shape
        s = self.scale.repeat_interleave(self.ws_rows, dim=0)[:N].repeat_interleave(GROUP, dim=1)[:, :K]
        return self.q.float() * s

    def rows(self, start: int, end: int) -> "Fp8Weight":
        assert start % self.ws_rows == 0 and (end % self.ws_rows == 0 or end == self.shape[0])
        return Fp8Weight(self.q[start:end], self.scale[start // self.ws_rows:_cdiv(end, self.ws_rows)], self.ws_rows)

    def nbytes(self) -> int:
        return self.q.numel() + self.scale.numel() * 4


def interleave_gate_up_fp8(gate: Fp8Weight, up: Fp8Weight, block: int = 32) -> Fp8Weight:
    """Row-interleave two [I, K] fp8 weights in blocks of 32 rows ([gate blk0 | up blk0 | gate blk1 | ...]) for
    the gated epilogue; the scales are expanded to one row per 32 weight rows."""
    I, K = gate.shape
    assert up.shape == gate.shape and I % block == 0 and gate.ws_rows % block == 0 and gate.ws_rows == up.ws_rows
    rep = gate.ws_rows // block
    gq = gate.q.view(torch.uint8).view(I // block, 1, block, K)
    uq = up.q.view(torch.uint8).view(I // block, 1, block, K)
    q = torch.cat([gq, uq], dim=1).reshape(2 * I, K).view(FP8)
    gs = gate.scale.repeat_interleave(rep, dim=0)[: I // block].unsqueeze(1)
    us = up.scale.repeat_interleave(rep, dim=0)[: I // block].unsqueeze(1)
    s = torch.cat([gs, us], dim=1).reshape(2 * (I // block), -1)
    return Fp8Weight(q, s, block)


def stack_experts(ws) -> Fp8Weight:
    """[E] x Fp8Weight [N, K] -> one Fp8Weight [E * N, K] (N a multiple of the scale granularity)."""
    g = ws[0].ws_rows
    assert all(w.ws_rows == g and w.shape == ws[0].shape and w.shape[0] % g == 0 for w in ws)
    return Fp8Weight(torch.cat([w.q.view(torch.uint8) for w in ws], 0).view(FP8), torch.cat([w.scale for w in ws], 0), g)


class Fp8Experts:
    """E expert matrices [N, K] stacked along the rows of one Fp8Weight (the grouped GEMM's weight operand)."""

    def __init__(self, stacked: Fp8Weight, E: int):
        assert stacked.shape[0] % E == 0
        self.w, self.E = stacked, E
        self.shape = (E, stacked.shape[0] // E, stacked.shape[1])
        self.device, self.dtype = stacked.device, torch.bfloat16

    def to(self, device) -> "Fp8Experts":
        return Fp8Experts(self.w.to(device), self.E)

    def dequant(self) -> torch.Tensor:
        return self.w.dequant().view(*self.shape)

    def nbytes(self) -> int:
        return self.w.nbytes()


def quant_act(x: torch.Tensor):
    """bf16 [M, K] -> (e4m3 [M, K], scale [ceil(K/128), M]).  CUDA: one warp per (token, group)."""
    if not x.is_cuda:
        return quant_act_reference(x)
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    M, K = x.shape
    q = torch.empty((M, K), dtype=FP8, device=x.device)
    s = torch.empty((_cdiv(K, GROUP), M), dtype=torch.float32, device=x.device)
    check(kernels().llb_quant_fp8_group128(ptr(x), i64(x.stride(0)), ptr(q), i64(K), ptr(s), i64(M), ctypes.c_int(M),
                                           ctypes.c_int(K), stream()), "quant_fp8_group128")
    _count()
    return q, s


def _epilogue_reference(acc, epi, residual):
    if epi == "gated_silu":
        M, N = acc.shape
        v = acc.view(M, N // 64, 2, 32)
        return (torch.nn.functional.silu(v[:, :, 0]) * v[:, :, 1]).reshape(M, N // 2)
    if epi == "residual":
        return acc + residual.float()
    return acc


def gemm_fp8_quantized(xq, xs, w: Fp8Weight, epi: str = "store", residual=None, out=None,
                       mblock_expert: Optional[torch.Tensor] = None, n_per_expert: Optional[int] = None):
    """C = (xq * xs) . (w.q * w.scale)^T.  Grouped mode (mblock_expert given): w stacks the experts, every
    128-row block i of xq multiplies with expert mblock_expert[i] (-1: skipped, output rows undefined)."""
    M, K = xq.shape
    N = n_per_expert if mblock_expert is not None else w.shape[0]
    n_out = N // 2 if epi == "gated_silu" else N
    if not xq.is_cuda:
        a = dequant_act(xq, xs)
        wd = w.dequant()
        if mblock_expert is None:
            acc = a @ wd.t()
        else:
            acc = torch.zeros(M, N, dtype=torch.float32)
            for i, e in enumerate(mblock_expert.tolist()):
                if e >= 0:
                    acc[i * 128:(i + 1) * 128] = a[i * 128:(i + 1) * 128] @ wd[e * N:(e + 1) * N].t()
        res = _epilogue_reference(acc, epi, residual).to(torch.bfloat16)
        if out is not None:
            out.copy_(res)
            return out
        return res
    from . import gemm_status

    assert xq.dtype == FP8 and xq.stride(1) == 1 and w.q.shape[1] == K and xs.shape[1] >= M
    if out is None:
        out = torch.empty((M, n_out), dtype=torch.bfloat16, device=xq.device)
    if epi == "residual":
        assert residual is not None and residual.shape == out.shape and residual.stride(0) == out.stride(0)
    check(kernels().llb_gemm_fp8_block(ptr(xq), i64(xq.stride(0)), ptr(xs), i64(xs.stride(0)), ptr(w.q), i64(K),
                                       ptr(w.scale), ctypes.c_int(w.ws_rows), ctypes.c_int(w.shape[0]), ptr(out),
                                       i64(out.stride(0)), ptr(residual), ctypes.c_int(M), ctypes.c_int(N),
                                       ctypes.c_int(K), ctypes.c_int(EPI[epi]), ptr(mblock_expert),
                                       ptr(gemm_status(xq.device)), stream()), "gemm_fp8_block")
    _count()
    return out


def gemm_fp8(a, w: Fp8Weight, epi: str = "store", residual=None, bias=None, out=None):
    """bf16 activations: quantise per token group, then the block-scaled GEMM.  epi "f32" returns fp32."""
    xq, xs = quant_act(a)
    kernel_epi = "store" if epi == "f32" else epi
    res = gemm_fp8_quantized(xq, xs, w, kernel_epi, residual, out if epi != "f32" else None)
    if bias is not None:
        res += bias
    if epi == "f32":
        res = res.float()
        if out is not None:
            out.copy_(res)
            return out
    return res
