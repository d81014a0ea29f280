"""int8 weights and activations (w8a8): one fp32 scale per output channel of the weight, one per token of the
activations, s32 accumulation on tcgen05 `kind::i8` (`csrc/gemm_fp8.cu`: gemm_i8_kernel); on CPU the same integer
arithmetic runs in torch.  Reference: lightllm/common/quantization/w8a8.py (method `w8a8` / `vllm-w8a8`).
"""
from __future__ import annotations

import ctypes

import torch

from . import _count
from ._native import check, i64, kernels, ptr, stream

EPI = {"store": 0, "residual": 1, "gated_silu": 2}


class Int8Weight:
    """[N, K] s8 weight with one fp32 scale per row (output channel)."""

    def __init__(self, q: torch.Tensor, scale: torch.Tensor):
        assert q.dtype == torch.int8 and q.dim() == 2 and scale.shape == (q.shape[0],)
        self.q, self.scale = q.contiguous(), scale.float().contiguous()
        self.shape = tuple(q.shape)
        self.device, self.dtype = q.device, torch.bfloat16

    @classmethod
    def from_float(cls, w: torch.Tensor) -> "Int8Weight":
        wf = w.float()
        s = wf.abs().amax(dim=1).clamp_min(1e-10) / 127.0
        q = torch.round(wf / s.unsqueeze(1)).clamp(-127, 127).to(torch.int8)
        return cls(q, s)

    def to(self, device) -> "Int8Weight":
        return Int8Weight(self.q.to(device), self.scale.to(device))

    def dequant(self) -> torch.Tensor:
        return self.q.float() * self.scale.unsqueeze(1)

    def nbytes(self) -> int:
        return self.q.numel() + self.scale.numel() * 4


def quant_act_reference(x: torch.Tensor):
    xf = x.float()
    s = xf.abs().amax(dim=1).clamp_min(1e-10) / 127.0
    q = torch.round(xf * (1.0 / s).unsqueeze(1)).clamp(-127, 127).to(torch.int8)
    return q, s


def quant_act(x: torch.Tensor):
    """bf16 [M, K] -> (s8 [M, K], scale [M]): symmetric, per token."""
    if not x.is_cuda:
        return quant_act_reference(x)
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    check(kernels().llb_quant_int8_per_token(ptr(x), i64(x.stride(0)), ptr(q), i64(K), ptr(s), ctypes.c_int(M),
                                             ctypes.c_int(K), stream()), "quant_int8_per_token")
    _count()
    return q, s


def gemm_int8_quantized(xq, xs, w: Int8Weight, epi: str = "store", residual=None, out=None):
    M, K = xq.shape
    N = w.shape[0]
    n_out = N // 2 if epi == "gated_silu" else N
    if not xq.is_cuda:
        acc = (xq.to(torch.int32) @ w.q.to(torch.int32).t()).float() * xs.unsqueeze(1) * w.scale.unsqueeze(0)
        if epi == "gated_silu":
            v = acc.view(M, N // 64, 2, 32)
            acc = (torch.nn.functional.silu(v[:, :, 0]) * v[:, :, 1]).reshape(M, N // 2)
        elif epi == "residual":
            acc = acc + residual.float()
        res = acc.to(torch.bfloat16)
        if out is not None:
            out.copy_(res)
            return out
        return res
    from . import gemm_status

    if out is None:
        out = torch.empty((M, n_out), dtype=torch.bfloat16, device=xq.device)
    if epi == "residual":
        assert residual is not None and residual.shape == out.shape and residual.stride(0) == out.stride(0)
    check(kernels().llb_gemm_int8(ptr(xq), i64(xq.stride(0)), ptr(xs), ptr(w.q), i64(K), ptr(w.scale), ptr(out),
                                  i64(out.stride(0)), ptr(residual), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
                                  ctypes.c_int(EPI[epi]), ptr(gemm_status(xq.device)), stream()), "gemm_int8")
    _count()
    return out


def gemm_int8(a, w: Int8Weight, epi: str = "store", residual=None, bias=None, out=None):
    xq, xs = quant_act(a)
    kernel_epi = "store" if epi == "f32" else epi
    res = gemm_int8_quantized(xq, xs, w, kernel_epi, residual, out if epi != "f32" else None)
    if bias is not None:
        res += bias
    if epi == "f32":
        res = res.float()
        if out is not None:
            out.copy_(res)
            return out
    return res
