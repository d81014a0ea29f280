"""int8 KV cache: storage layout, quantising store, and attention over the quantised pool.

A (slot, head) row of the pool is `D` int8 values followed by one fp32 scale and 12 unused bytes (x = q * scale,
scale = max|x| / 127 over the row), so a token's row is an opaque byte string for everything that moves KV around.
`Int8KVLayer` wraps one layer's slice of the pool; the attention ops accept it wherever they take a bf16 slice:

* new K / V rows are rotated into a scratch tensor and quantised into their slots (`quant_store_`);
* decode attention reads the int8 rows directly (`csrc/attention_int8kv.cu`);
* prefill (and the generic-head-size kernel) runs on a bf16 copy of the rows the batch refers to, gathered and
  widened once per layer, with a request table that points into that copy.

The fp8 pool (`Fp8KVLayer`, `--llm_kv_type fp8kv_sph | fp8kv_spt`) stores e4m3 rows without a scale in the row: the
scales are static numbers per (layer, head) -- or one per layer for K and one for V -- read from a calibration file
(`--kv_quant_calibration_config_path`; ones without a file).  The same three routes apply.

Reference: lightllm/common/kv_cache_mem_manager/ppl_int8kv_mem_manager.py, fp8_static_per_head_quant_mem_manager.py,
fp8_static_per_tensor_quant_mem_manager.py, common/basemodel/attention/triton/int8kv.py, attention/fa3/fp8.py,
`--llm_kv_type`.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

PAD = 16  # bytes after the payload of a row: fp32 scale + padding


class QuantKVLayer:
    """A layer of a quantised pool; the attention ops accept it in place of a bf16 slice."""

    __slots__ = ()


class Fp8KVLayer(QuantKVLayer):
    """`data` e4m3 (stored as uint8) [slots + 1, 2 * Hkv, D]; `scales` fp32 [2 * Hkv] (K heads, then V heads)."""

    __slots__ = ("data", "head_dim", "scales")

    def __init__(self, data: torch.Tensor, head_dim: int, scales: torch.Tensor):
        assert data.dtype == torch.uint8 and data.shape[-1] == head_dim and scales.shape[0] == data.shape[1]
        self.data, self.head_dim, self.scales = data, head_dim, scales

    @property
    def device(self):
        return self.data.device

    @property
    def is_cuda(self):
        return self.data.is_cuda

    def _deq(self, rows, dtype):
        return (rows.view(torch.float8_e4m3fn).float() * self.scales.view(1, -1, 1)).to(dtype)

    def dequant_rows(self, slots: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        return self._deq(self.data.index_select(0, slots.to(self.data.device, torch.long)), dtype)

    def dequant_all(self, dtype: torch.dtype) -> torch.Tensor:
        return self._deq(self.data, dtype)

    def store_(self, src: torch.Tensor, slot: torch.Tensor) -> None:
        q = (src.float() / self.scales.view(1, -1, 1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
        self.data[slot.long()] = q.view(torch.uint8)


class CalibratingKVLayer(QuantKVLayer):
    """A bf16 layer that records the largest |value| per head of everything stored into it (used to make the scale
    file of the fp8 pools): `data` [slots + 1, 2 * Hkv, D] in the compute dtype, `amax` fp32 [2 * Hkv]."""

    __slots__ = ("data", "head_dim", "amax")

    def __init__(self, data: torch.Tensor, head_dim: int, amax: torch.Tensor):
        self.data, self.head_dim, self.amax = data, head_dim, amax

    @property
    def device(self):
        return self.data.device

    @property
    def is_cuda(self):
        return self.data.is_cuda

    def dequant_rows(self, slots, dtype):
        return self.data.index_select(0, slots.to(self.data.device, torch.long)).to(dtype)

    def dequant_all(self, dtype):
        return self.data.to(dtype)

    def store_(self, src, slot):
        torch.maximum(self.amax, src.float().abs().amax(dim=(0, 2)), out=self.amax)
        self.data[slot.long()] = src.to(self.data.dtype)


class Int8KVLayer(QuantKVLayer):
    """One layer of the quantised pool: `data` int8 [slots + 1, 2 * Hkv, D + 16]."""

    __slots__ = ("data", "head_dim")

    def __init__(self, data: torch.Tensor, head_dim: int):
        assert data.dtype == torch.int8 and data.shape[-1] == head_dim + PAD
        self.data = data
        self.head_dim = head_dim

    @property
    def device(self):
        return self.data.device

    @property
    def is_cuda(self):
        return self.data.is_cuda

    def scales(self, rows: torch.Tensor) -> torch.Tensor:
        """fp32 scales [..., 1] of already gathered rows [..., D + 16]."""
        D = self.head_dim
        return rows[..., D:D + 4].contiguous().view(torch.float32)

    def dequant_rows(self, slots: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        """[n, 2 * Hkv, D] in `dtype` for the given slots."""
        rows = self.data.index_select(0, slots.to(self.data.device, torch.long))
        return (rows[..., : self.head_dim].float() * self.scales(rows)).to(dtype)

    def dequant_all(self, dtype: torch.dtype) -> torch.Tensor:
        return (self.data[..., : self.head_dim].float() * self.scales(self.data)).to(dtype)


class Int4KVLayer(QuantKVLayer):
    """One layer of the 4-bit pool: `data` uint8 [slots + 1, 2 * Hkv, D / 2 + 2 * D / group]: two values per byte
    (low nibble first, stored as value + 8), then one fp16 scale per `group` consecutive values (x = q * scale,
    scale = max|x| / 7 over the group).  Attention runs on a widened copy of the rows a batch refers to.
    Reference: lightllm/common/kv_cache_mem_manager/ppl_int4kv_mem_manager.py (`--llm_kv_type int4kv`,
    `--llm_kv_quant_group_size`)."""

    __slots__ = ("data", "head_dim", "group")

    def __init__(self, data: torch.Tensor, head_dim: int, group: int):
        assert data.dtype == torch.uint8 and head_dim % group == 0 and group % 2 == 0
        assert data.shape[-1] == self.row_bytes(head_dim, group)
        self.data, self.head_dim, self.group = data, head_dim, group

    @staticmethod
    def row_bytes(head_dim: int, group: int) -> int:
        return head_dim // 2 + 2 * (head_dim // group)

    @property
    def device(self):
        return self.data.device

    @property
    def is_cuda(self):
        return self.data.is_cuda

    def _deq(self, rows: torch.Tensor, dtype) -> torch.Tensor:
        D, g = self.head_dim, self.group
        packed = rows[..., : D // 2]
        lo = (packed & 0xF).to(torch.int16) - 8
        hi = (packed >> 4).to(torch.int16) - 8
        q = torch.stack([lo, hi], dim=-1).reshape(*rows.shape[:-1], D // g, g).float()
        scale = rows[..., D // 2:].contiguous().view(torch.float16).float().unsqueeze(-1)
        return (q * scale).reshape(*rows.shape[:-1], D).to(dtype)

    def dequant_rows(self, slots: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        return self._deq(self.data.index_select(0, slots.to(self.data.device, torch.long)), dtype)

    def dequant_all(self, dtype: torch.dtype) -> torch.Tensor:
        return self._deq(self.data, dtype)

    def store_(self, src: torch.Tensor, slot: torch.Tensor) -> None:
        D, g = self.head_dim, self.group
        x = src.float().reshape(*src.shape[:-1], D // g, g)
        amax = x.abs().amax(dim=-1, keepdim=True)
        scale = torch.where(amax > 0, amax / 7.0, torch.ones_like(amax)).to(torch.float16)
        q = torch.clamp(torch.round(x / scale.float()), -7, 7).to(torch.int16) + 8
        q = q.reshape(*src.shape[:-1], D // 2, 2)
        packed = (q[..., 0] | (q[..., 1] << 4)).to(torch.uint8)
        row = torch.cat([packed, scale.squeeze(-1).contiguous().view(torch.uint8)], dim=-1)
        self.data[slot.long()] = row


def quant_rows_reference(x: torch.Tensor):
    """x [..., D] -> (int8 [..., D], fp32 scale [..., 1]); the definition the CUDA kernel is checked against."""
    xf = x.float()
    amax = xf.abs().amax(dim=-1, keepdim=True)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    q = torch.clamp(torch.round(xf / scale), -127, 127).to(torch.int8)
    return q, scale


def quant_store_(layer, src: torch.Tensor, slot: torch.Tensor) -> None:
    """layer[slot[t]] = quantised src[t];  src [T, 2 * Hkv, D] (bf16 on the GPU)."""
    if isinstance(layer, (Fp8KVLayer, CalibratingKVLayer, Int4KVLayer)):
        return layer.store_(src, slot)
    T, rows, D = src.shape
    assert D == layer.head_dim and rows == layer.data.shape[1]
    if not src.is_cuda:
        q, scale = quant_rows_reference(src)
        packed = torch.zeros((T, rows, D + PAD), dtype=torch.int8)
        packed[..., :D] = q
        packed[..., D:D + 4] = scale.contiguous().view(torch.int8)
        layer.data[slot.long()] = packed
        return
    from . import _count, c_int, check, i64, kernels, ptr, stream

    assert src.dtype == torch.bfloat16 and src.stride(2) == 1 and src.stride(1) == D and slot.dtype == torch.int32
    check(kernels().llb_kv_quant_store_int8(ptr(src), i64(src.stride(0)), ptr(layer.data), ptr(slot), c_int(T),
                                            c_int(rows), c_int(D), stream()), "kv_quant_store_int8")
    _count()


def rope_kv_scatter_(qkv, layer, cos, sin, pos, slot, Hq, Hkv, D, *rest, **kw):
    """The rotary / norm / scatter op with a quantised destination: K and V go through a scratch tensor."""
    from . import rope_kv_scatter_ as plain

    T = qkv.shape[0]
    tmp = torch.empty((T, 2 * Hkv, D), dtype=qkv.dtype, device=qkv.device)
    ident = torch.arange(T, dtype=torch.int32, device=qkv.device)
    plain(qkv, tmp, cos, sin, pos, ident, Hq, Hkv, D, *rest, **kw)
    quant_store_(layer, tmp, slot)
    return qkv


def gqa_decode(q, layer, req_to_token, b_req_idx, b_seq_len, Hq, Hkv, D, max_seq_len, sm_scale=None,
               out=None, num_splits: Optional[int] = None, scratch=None):
    from . import _count, _scratch, c_int, check, f32, gqa_decode as plain, gqa_decode_num_splits, i64, kernels, ptr, \
        stream

    if isinstance(layer, CalibratingKVLayer):
        return plain(q, layer.data, req_to_token, b_req_idx, b_seq_len, Hq, Hkv, D, max_seq_len, sm_scale, out,
                     num_splits, scratch)
    if not q.is_cuda or D not in (64, 128) or isinstance(layer, Int4KVLayer):
        if not q.is_cuda:
            return plain(q, layer.dequant_all(q.dtype), req_to_token, b_req_idx, b_seq_len, Hq, Hkv, D, max_seq_len,
                         sm_scale)
        kv, r2t, idx = gather_dequant(layer, req_to_token, b_req_idx, b_seq_len, q.dtype)
        return plain(q, kv, r2t, idx, b_seq_len, Hq, Hkv, D, max_seq_len, sm_scale, out=out, num_splits=num_splits,
                     scratch=scratch)
    B = q.shape[0]
    assert q.dtype == torch.bfloat16 and q.stride(-1) == 1 and layer.data.is_contiguous()
    scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty((B, Hq, D), dtype=q.dtype, device=q.device)
    if num_splits is None:
        num_splits = gqa_decode_num_splits(B, Hq, Hkv, max_seq_len)
    po = pl = None
    if num_splits > 1:
        po, pl = scratch if scratch is not None else _scratch(q.device, B * Hq * num_splits * D, B * Hq * num_splits)
    if isinstance(layer, Fp8KVLayer):
        check(kernels().llb_gqa_decode_fp8kv(ptr(q), i64(q.stride(0)), ptr(layer.data), ptr(req_to_token),
                                             i64(req_to_token.stride(0)), ptr(b_req_idx), ptr(b_seq_len), ptr(out),
                                             i64(out.stride(0)), ptr(po), ptr(pl), c_int(B), c_int(Hq), c_int(Hkv),
                                             c_int(D), c_int(num_splits), f32(scale), ptr(layer.scales), stream()),
              "gqa_decode_fp8kv")
        _count(2 if num_splits > 1 else 1)
        return out
    check(kernels().llb_gqa_decode_int8kv(ptr(q), i64(q.stride(0)), ptr(layer.data), ptr(req_to_token),
                                          i64(req_to_token.stride(0)), ptr(b_req_idx), ptr(b_seq_len), ptr(out),
                                          i64(out.stride(0)), ptr(po), ptr(pl), c_int(B), c_int(Hq), c_int(Hkv),
                                          c_int(D), c_int(num_splits), f32(scale), stream()), "gqa_decode_int8kv")
    _count(2 if num_splits > 1 else 1)
    return out


def gather_dequant(layer, req_to_token, b_req_idx, b_seq_len, dtype):
    """A bf16 copy of the rows the batch refers to: (kv [n + 1, 2 * Hkv, D], request table [B, max_len] into it,
    request ids 0 .. B - 1).  Row n is a zero row for the positions past a request's length."""
    dev = layer.data.device
    B = b_req_idx.shape[0]
    lens = b_seq_len.to(dev, torch.long)
    max_len = int(lens.max().item()) if B else 0
    table = req_to_token.index_select(0, b_req_idx.to(dev, torch.long))[:, :max_len].to(torch.long)
    valid = torch.arange(max_len, device=dev)[None, :] < lens[:, None]
    slots = table[valid]
    kv = torch.zeros((slots.shape[0] + 1, layer.data.shape[1], layer.head_dim), dtype=dtype, device=dev)
    kv[:-1] = layer.dequant_rows(slots, dtype)
    new_table = torch.full((B, max(max_len, 1)), slots.shape[0], dtype=torch.int32, device=dev)
    new_table[:, :max_len][valid] = torch.arange(slots.shape[0], dtype=torch.int32, device=dev)
    return kv, new_table, torch.arange(B, dtype=torch.int32, device=dev)


def gqa_prefill(q, layer, req_to_token, b_req_idx, cu_q, b_ready_len, Hq, Hkv, D, max_q_len,
                sm_scale=None, out=None):
    from . import gqa_prefill as plain

    if isinstance(layer, CalibratingKVLayer):
        return plain(q, layer.data, req_to_token, b_req_idx, cu_q, b_ready_len, Hq, Hkv, D, max_q_len, sm_scale, out)

    lens = b_ready_len.to(layer.device) + (cu_q[1:] - cu_q[:-1]).to(layer.device)
    kv, r2t, idx = gather_dequant(layer, req_to_token, b_req_idx, lens.to(torch.int32), q.dtype)
    return plain(q, kv, r2t, idx, cu_q, b_ready_len, Hq, Hkv, D, max_q_len, sm_scale, out)


def attention_generic(q, layer, req_to_token, b_req_idx, pos, batch_of, Hq, Hkv, D, sm_scale, *rest, **kw):
    from . import attention_generic as plain

    if isinstance(layer, CalibratingKVLayer):
        return plain(q, layer.data, req_to_token, b_req_idx, pos, batch_of, Hq, Hkv, D, sm_scale, *rest, **kw)
    dev = layer.device
    B = b_req_idx.shape[0]
    p = pos.to(dev, torch.long)
    if batch_of is None:   # decode: one token per request
        lens = p + 1
    else:
        lens = torch.zeros(B, dtype=torch.long, device=dev).scatter_reduce_(0, batch_of.to(dev, torch.long), p + 1,
                                                                             reduce="amax")
    kv, r2t, idx = gather_dequant(layer, req_to_token, b_req_idx, lens.to(torch.int32), q.dtype)
    return plain(q, kv, r2t, idx, pos, batch_of, Hq, Hkv, D, sm_scale, *rest, **kw)
