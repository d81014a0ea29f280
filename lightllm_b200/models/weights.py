"""Checkpoint access: HF safetensors directories (bf16 / fp16, fp8 e4m3 with `weight_scale_inv`
128x128 block scales) and a deterministic random-init source of the same names/shapes.

A model asks a `WeightSource` for tensors by HF name, optionally sliced along one dim (the
tensor-parallel rules: row slicing = split `out` (dim 0) for q/k/v/gate/up/lm_head, column
slicing = split `in` (dim 1) for o_proj/down_proj; block scales are sliced with the same rule
at 1/128 granularity).  Reference: lightllm/common/basemodel/layer_weights/hf_load_utils.py:31-72
and meta_weights/mm_weight/mm_slicer.py.
"""
from __future__ import annotations

import glob
import hashlib
import json
import os
from typing import Dict, Optional, Sequence

import torch


class WeightSource:
    def has(self, name: str) -> bool:
        raise NotImplementedError

    def get(self, name: str, dim: Optional[int] = None, start: int = 0, end: Optional[int] = None) -> torch.Tensor:
        """Tensor `name` on CPU (or generated on `self.device`), optionally sliced [start:end) along dim."""
        raise NotImplementedError

    def shape(self, name: str):
        raise NotImplementedError

    def names(self) -> Sequence[str]:
        raise NotImplementedError


class SafetensorsSource(WeightSource):
    """Lazy reader over every *.safetensors of a model directory (falls back to *.bin)."""

    def __init__(self, model_dir: str):
        from safetensors import safe_open

        self.model_dir = model_dir
        self._open = safe_open
        self._file_of: Dict[str, str] = {}
        self._handles = {}
        idx = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                for k, v in json.load(f)["weight_map"].items():
                    self._file_of[k] = os.path.join(model_dir, v)
        else:
            files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
            for fp in files:
                with safe_open(fp, framework="pt", device="cpu") as f:
                    for k in f.keys():
                        self._file_of[k] = fp
        self._bin: Dict[str, torch.Tensor] = {}
        if not self._file_of:
            for fp in sorted(glob.glob(os.path.join(model_dir, "*.bin"))):
                self._bin.update(torch.load(fp, map_location="cpu", weights_only=True))

    def _h(self, fp):
        if fp not in self._handles:
            self._handles[fp] = self._open(fp, framework="pt", device="cpu")
        return self._handles[fp]

    def has(self, name):
        return name in self._file_of or name in self._bin

    def names(self):
        return list(self._file_of.keys()) + list(self._bin.keys())

    def shape(self, name):
        if name in self._bin:
            return tuple(self._bin[name].shape)
        return tuple(self._h(self._file_of[name]).get_slice(name).get_shape())

    def get(self, name, dim=None, start=0, end=None):
        if name in self._bin:
            t = self._bin[name]
            if dim is not None:
                t = t.narrow(dim, start, (end if end is not None else t.shape[dim]) - start)
            return t
        h = self._h(self._file_of[name])
        if dim is None:
            return h.get_tensor(name)
        sl = h.get_slice(name)
        nd = len(sl.get_shape())
        end = sl.get_shape()[dim] if end is None else end
        index = tuple(slice(start, end) if d == dim else slice(None) for d in range(nd))
        return sl[index]


class RandomSource(WeightSource):
    """Deterministic N(0, std) tensors keyed by name: every rank that asks for a name sees the same
    full tensor, so TP=n output can be checked against TP=1.  Norm weights are ones.  fp8 weights
    are generated as e4m3 payload ~ N(0, 96) plus `*_scale_inv` ~ U(0.5, 2) * std / 96 block scales."""

    def __init__(self, shapes: Dict[str, tuple], dtype=torch.bfloat16, std: float = 0.02, seed: int = 0,
                 device: str = "cpu", fp8_names: Optional[set] = None):
        self.shapes = dict(shapes)
        self.dtype = dtype
        self.std = std
        self.seed = seed
        self.device = torch.device(device)
        self.fp8_names = fp8_names or set()

    def has(self, name):
        return name in self.shapes

    def names(self):
        return list(self.shapes.keys())

    def shape(self, name):
        return tuple(self.shapes[name])

    def _gen(self, name):
        h = int.from_bytes(hashlib.sha256(f"{self.seed}:{name}".encode()).digest()[:7], "little")
        g = torch.Generator(device=self.device)
        g.manual_seed(h)
        return g

    def get(self, name, dim=None, start=0, end=None):
        shape = self.shapes[name]
        if name.endswith("norm.weight") or name.endswith("layernorm.weight") or name.endswith("_norm.weight") or \
                name.endswith("layer_scalar") or name.endswith("router.scale") or name.endswith("per_expert_scale"):
            t = torch.ones(shape, dtype=self.dtype, device=self.device)
        elif name.endswith("_scale_inv"):
            t = (torch.rand(shape, generator=self._gen(name), device=self.device, dtype=torch.float32) * 1.5 + 0.5) * (self.std / 96.0)
        elif name in self.fp8_names:
            t = (torch.randn(shape, generator=self._gen(name), device=self.device, dtype=torch.float32) * 96.0)
            t = t.clamp(-448, 448).to(torch.float8_e4m3fn)
        elif name.endswith("e_score_correction_bias"):
            t = torch.zeros(shape, dtype=torch.float32, device=self.device)
        else:
            t = torch.randn(shape, generator=self._gen(name), device=self.device, dtype=torch.float32) * self.std
            t = t.to(self.dtype)
        if dim is not None:
            end = shape[dim] if end is None else end
            t = t.narrow(dim, start, end - start)
        return t


def tp_range(total: int, tp_rank: int, tp_size: int):
    """Even split [start, end) of `total` items for a rank (total must divide)."""
    assert total % tp_size == 0, f"{total} not divisible by tp {tp_size}"
    per = total // tp_size
    return tp_rank * per, (tp_rank + 1) * per


def kv_head_range(num_kv_heads: int, tp_rank: int, tp_size: int):
    """KV heads of a rank; heads are replicated when tp > kv heads
    (lightllm/common/basemodel/layer_weights/meta_weights/mm_weight/rowmm_weight.py:76-88)."""
    if tp_size <= num_kv_heads:
        return tp_range(num_kv_heads, tp_rank, tp_size)
    rep = tp_size // num_kv_heads
    h = tp_rank // rep
    return h, h + 1
