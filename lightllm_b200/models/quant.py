"""Weight quantisation formats of checkpoints.

fp8 block format (DeepSeek-V3 style): `X.weight` is float8_e4m3fn [out, in] and `X.weight_scale_inv` is
fp32 [ceil(out/128), ceil(in/128)]; the real weight is weight * scale_inv broadcast over 128x128 blocks.
TP slicing applies the same row/column rule to the scale tensor at 1/128 granularity, so sharded
dimensions must be multiples of 128 (reference: mm_slicer.py Quantized*SliceMixin, deepgemm.py:46-56).

`load_dequant` returns the bf16 weight of a slice (the block-dequantising load path);
`load_fp8` returns (e4m3 payload, scales) for the block-scaled fp8 GEMM.
"""
from __future__ import annotations

from typing import Optional

import torch

BLOCK = 128


def is_fp8_block_config(cfg: dict) -> bool:
    q = cfg.get("quantization_config") or {}
    return q.get("quant_method") == "fp8" and list(q.get("weight_block_size") or []) == [BLOCK, BLOCK]


def _scale_slice(src, name, dim, start, end):
    sname = name + "_scale_inv"
    if dim is None:
        return src.get(sname)
    assert start % BLOCK == 0, f"fp8 block-quantised {name}: slice start {start} is not a multiple of {BLOCK}"
    s0 = start // BLOCK
    s1 = None if end is None else (end + BLOCK - 1) // BLOCK
    return src.get(sname, dim, s0, s1)


def dequant_block(w: torch.Tensor, scale_inv: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    out_f, in_f = w.shape
    s = scale_inv.float().repeat_interleave(BLOCK, 0)[:out_f].repeat_interleave(BLOCK, 1)[:, :in_f]
    return (w.float() * s).to(dtype)


def quant_block(w: torch.Tensor):
    """bf16/fp32 [out, in] -> (e4m3 payload, scale_inv) with one scale per 128x128 block (online quantisation)."""
    out_f, in_f = w.shape
    po, pi = (out_f + BLOCK - 1) // BLOCK, (in_f + BLOCK - 1) // BLOCK
    wp = torch.zeros(po * BLOCK, pi * BLOCK, dtype=torch.float32, device=w.device)
    wp[:out_f, :in_f] = w.float()
    blocks = wp.view(po, BLOCK, pi, BLOCK)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / 448.0
    q = (blocks / scale[:, None, :, None]).clamp(-448, 448).view(po * BLOCK, pi * BLOCK)[:out_f, :in_f]
    return q.to(torch.float8_e4m3fn), scale


def load_dequant(src, name: str, dim: Optional[int] = None, start: int = 0, end: Optional[int] = None,
                 dtype=torch.bfloat16) -> torch.Tensor:
    w = src.get(name, dim, start, end) if dim is not None else src.get(name)
    if w.dtype == torch.float8_e4m3fn and src.has(name + "_scale_inv"):
        return dequant_block(w, _scale_slice(src, name, dim, start, end), dtype)
    return w


def load_fp8(src, name: str, dim: Optional[int] = None, start: int = 0, end: Optional[int] = None):
    w = src.get(name, dim, start, end) if dim is not None else src.get(name)
    if w.dtype == torch.float8_e4m3fn:
        return w, _scale_slice(src, name, dim, start, end).float()
    return quant_block(w)


def load_fp8_weight(src, name: str, dim: Optional[int] = None, start: int = 0, end: Optional[int] = None):
    """Fp8Weight (e4m3 payload + 128 x 128 block scales) of a checkpoint tensor slice; bf16 checkpoints are
    quantised on the fly (`--quant_type fp8w8a8-b128` on an unquantised model)."""
    from ..ops.fp8 import Fp8Weight

    q, s = load_fp8(src, name, dim, start, end)
    return Fp8Weight(q.contiguous(), s.contiguous().float(), BLOCK)


class DequantSource:
    """WeightSource view that hands out bf16 tensors for fp8 block-quantised entries."""

    def __init__(self, base, dtype=torch.bfloat16):
        self.base, self.dtype = base, dtype

    def has(self, n):
        return self.base.has(n)

    def shape(self, n):
        return self.base.shape(n)

    def names(self):
        return self.base.names()

    def get(self, n, dim=None, start=0, end=None):
        return load_dequant(self.base, n, dim, start, end, self.dtype)


# ---- AWQ (4-bit weight-only, AutoAWQ "GEMM" packing) ----
# `X.qweight` int32 [K, N/8] holds eight 4-bit values per word in the order 0, 2, 4, 6, 1, 3, 5, 7 (value j of a
# word sits at bits 4 * AWQ_ORDER.index(j)), `X.qzeros` int32 [K/g, N/8] the zero points in the same packing,
# `X.scales` fp16 [K/g, N]; the weight is W[n, k] = (q[k, n] - z[k / g, n]) * s[k / g, n].  There is no int4 GEMM in
# this build: such checkpoints are expanded to bf16 at load (reference: lightllm/common/quantization/awq.py runs
# them through vllm's awq / marlin kernels).
_AWQ_REVERSE = (0, 4, 1, 5, 2, 6, 3, 7)


def awq_unpack(packed: torch.Tensor) -> torch.Tensor:
    """int32 [R, C/8] -> int32 [R, C] of 4-bit values in natural column order."""
    shifts = torch.arange(0, 32, 4, device=packed.device, dtype=torch.int32)
    v = (packed.unsqueeze(-1) >> shifts) & 0xF                      # [R, C/8, 8] in packed order
    v = v[:, :, list(_AWQ_REVERSE)]
    return v.reshape(packed.shape[0], -1)


def awq_pack(values: torch.Tensor) -> torch.Tensor:
    """Inverse of `awq_unpack` (used by tests and by tools that write checkpoints)."""
    R, C = values.shape
    v = values.to(torch.int32).view(R, C // 8, 8)
    order = (0, 2, 4, 6, 1, 3, 5, 7)
    out = torch.zeros(R, C // 8, dtype=torch.int32, device=values.device)
    for pos, j in enumerate(order):
        out |= (v[:, :, j] & 0xF) << (4 * pos)
    return out


def awq_dequant(qweight, qzeros, scales, dtype=torch.bfloat16) -> torch.Tensor:
    """-> [N, K] weight in the checkpoint layout of an unquantised Linear."""
    q = awq_unpack(qweight)                   # [K, N]
    z = awq_unpack(qzeros)                    # [K/g, N]
    g = q.shape[0] // z.shape[0]
    w = (q - z.repeat_interleave(g, dim=0)).float() * scales.float().repeat_interleave(g, dim=0)
    return w.t().contiguous().to(dtype)


class AwqDequantSource:
    """WeightSource view of an AWQ checkpoint: `X.weight` is built from `X.qweight / qzeros / scales`."""

    def __init__(self, base, dtype=torch.bfloat16):
        self.base, self.dtype = base, dtype
        self._last = (None, None)

    def _q(self, n):
        return n.endswith(".weight") and not self.base.has(n) and self.base.has(n[:-len("weight")] + "qweight")

    def has(self, n):
        return self.base.has(n) or self._q(n)

    def names(self):
        out = []
        for n in self.base.names():
            if n.endswith(".qweight"):
                out.append(n[:-len("qweight")] + "weight")
            elif not (n.endswith(".qzeros") or n.endswith(".scales")):
                out.append(n)
        return out

    def _full(self, n):
        if self._last[0] != n:
            p = n[:-len("weight")]
            self._last = (n, awq_dequant(self.base.get(p + "qweight"), self.base.get(p + "qzeros"),
                                         self.base.get(p + "scales"), self.dtype))
        return self._last[1]

    def shape(self, n):
        if self._q(n):
            p = n[:-len("weight")]
            k, n8 = self.base.shape(p + "qweight")
            return (n8 * 8, k)
        return self.base.shape(n)

    def get(self, n, dim=None, start=0, end=None):
        if not self._q(n):
            return self.base.get(n, dim, start, end)
        t = self._full(n)
        if dim is not None:
            end = t.shape[dim] if end is None else end
            t = t.narrow(dim, start, end - start)
        return t
