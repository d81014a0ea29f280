"""Checkpoint name translation.  `RemapSource` presents a checkpoint under the canonical Llama-style names the
model classes read (`model.layers.N.self_attn.q_proj.weight`, ...): an entry is either the checkpoint's own name
or a function that builds the tensor (splitting a fused qkv / gate_up tensor, undoing a per-head interleave).
Reference: the per-family `pre_and_post_layer_weight.py` / `transformer_layer_weight.py` files of lightllm/models/*.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Union

import torch

from .weights import WeightSource

Entry = Union[str, Callable[[WeightSource], torch.Tensor]]


class RemapSource(WeightSource):
    def __init__(self, base: WeightSource, table: Dict[str, Entry], passthrough: bool = True):
        self.base, self.table, self.passthrough = base, table, passthrough
        self._cache: Dict[str, torch.Tensor] = {}

    def has(self, name):
        e = self.table.get(name)
        if e is None:
            return self.passthrough and self.base.has(name)
        if isinstance(e, str):
            return self.base.has(e)
        return True

    def names(self):
        return list(self.table.keys())

    def _full(self, name):
        e = self.table.get(name)
        if e is None:
            return None
        if isinstance(e, str):
            return None
        t = self._cache.get(name)
        if t is None:
            t = e(self.base)
            self._cache = {name: t}  # one entry: split products of a fused tensor are asked for back to back
        return t

    def get(self, name, dim: Optional[int] = None, start: int = 0, end: Optional[int] = None):
        e = self.table.get(name)
        if e is None:
            return self.base.get(name, dim, start, end)
        if isinstance(e, str):
            return self.base.get(e, dim, start, end)
        t = self._full(name)
        if dim is not None:
            end = t.shape[dim] if end is None else end
            t = t.narrow(dim, start, end - start)
        return t

    def shape(self, name):
        e = self.table.get(name)
        if e is None:
            return self.base.shape(name)
        if isinstance(e, str):
            return self.base.shape(e)
        return tuple(self._full(name).shape)


def split_rows(fused_name: str, start: int, end: int, suffix: str = "") -> Callable[[WeightSource], torch.Tensor]:
    """Rows [start, end) of a fused tensor (works for weights [out, in] and biases [out])."""
    return lambda src: src.get(fused_name + suffix, 0, start, end)


def per_head_qkv(fused_name: str, num_heads: int, head_dim: int, which: int) -> Callable[[WeightSource], torch.Tensor]:
    """Bloom-style fused qkv laid out [head][q|k|v][head_dim] along the rows: the rows of q (which=0), k (1) or v (2)
    for all heads."""
    def f(src):
        t = src.get(fused_name)
        t = t.view(num_heads, 3, head_dim, *t.shape[1:])
        return t[:, which].reshape(num_heads * head_dim, *t.shape[3:])

    return f


def grouped_qkv(fused_name: str, num_kv: int, group: int, head_dim: int, which: str):
    """InternLM2-style wqkv laid out [kv head][group q heads | k | v][head_dim]."""
    def f(src):
        t = src.get(fused_name)
        t = t.view(num_kv, group + 2, head_dim, t.shape[-1])
        if which == "q":
            return t[:, :group].reshape(num_kv * group * head_dim, -1)
        if which == "k":
            return t[:, group].reshape(num_kv * head_dim, -1)
        return t[:, group + 1].reshape(num_kv * head_dim, -1)

    return f


class FusedExperts:
    """Per-expert views of expert weights stored as one 3-D tensor [E, out, in] (or [E, in, out] in older
    checkpoints, recognised by `out_features`); the tensor is fetched once and kept while its experts are read."""

    def __init__(self):
        self._name, self._t = None, None

    def _load(self, src, name, out_features):
        if self._name != name:
            t = src.get(name)
            if t.shape[1] != out_features and t.shape[2] == out_features:
                t = t.transpose(1, 2)
            self._name, self._t = name, t
        return self._t

    def entry(self, name: str, expert: int, out_features: int, r0: int = 0, r1: Optional[int] = None):
        def f(src):
            t = self._load(src, name, out_features)[expert]
            return t[r0:r1].contiguous()

        return f
