"""Routed-expert capture (`--enable_return_routed_experts`): which experts every token went to, per MoE layer.

The model keeps `routing[kv_slot, moe_layer, top_k]` on the device, indexed by the token's KV slot, so tokens that
come out of the prefix cache bring their routing with them.  A MoE layer scatters the router's top-k ids of the
tokens of the pass into it (one small kernel, graph-safe: the slot numbers come from the step's static buffer).
When a request finishes, the rows of its slots are gathered and copied to the host, written to a shared-memory
array of the request, and the HTTP worker returns them as {"shape", "dtype", "data" (base64 of the C-order bytes)}.
Ids are uint8 for up to 256 experts, else int16.

Reference: lightllm/common/basemodel/moe_route_info_manager.py:1-263 (pinned host buffer written by a Triton
scatter; here the buffer stays in HBM and is read once per finished request),
lightllm/server/core/objs/token_metadata.py:159-176 (response encoding).
"""
from __future__ import annotations

import base64
import ctypes
from typing import Dict, Optional

import numpy as np
import torch


def text_config(config: dict) -> dict:
    return config.get("text_config", config) if isinstance(config.get("text_config"), dict) else config


def num_experts_of(config: dict) -> int:
    c = text_config(config)
    return int(c.get("n_routed_experts") or c.get("num_experts") or c.get("num_local_experts") or 0)


def moe_layer_map(config: dict) -> Dict[int, int]:
    """transformer layer index -> dense index among the MoE layers."""
    c = text_config(config)
    n = int(c.get("num_hidden_layers") or c.get("n_layer") or c.get("num_layers") or 0)
    if num_experts_of(c) <= 0 or n <= 0:
        return {}
    if "first_k_dense_replace" in c:
        first, freq = int(c.get("first_k_dense_replace", 0)), int(c.get("moe_layer_freq", 1) or 1)
        layers = [i for i in range(n) if i >= first and i % freq == 0]
    elif "mlp_only_layers" in c or "decoder_sparse_step" in c:
        only, step = set(c.get("mlp_only_layers") or []), int(c.get("decoder_sparse_step", 1) or 1)
        layers = [i for i in range(n) if i not in only and (i + 1) % step == 0]
    else:
        layers = list(range(n))
    return {layer: j for j, layer in enumerate(layers)}


def top_k_of(config: dict) -> int:
    c = text_config(config)
    return int(c.get("num_experts_per_tok") or c.get("top_k_experts") or 0)


def np_dtype_of(config: dict):
    return np.uint8 if num_experts_of(config) <= 256 else np.int16


def encode(arr: Optional[np.ndarray]) -> Optional[dict]:
    if arr is None:
        return None
    arr = np.ascontiguousarray(arr)
    return {"shape": list(arr.shape), "dtype": str(arr.dtype), "data": base64.b64encode(arr.tobytes()).decode("ascii")}


def decode(obj: dict) -> np.ndarray:
    return np.frombuffer(base64.b64decode(obj["data"]), dtype=np.dtype(obj["dtype"])).reshape(obj["shape"])


class RouteCapture:
    def __init__(self, config: dict, kv_slots: int, device):
        self.layer_map = moe_layer_map(config)
        self.top_k = top_k_of(config)
        assert self.layer_map and self.top_k > 0, "--enable_return_routed_experts needs a mixture-of-experts model"
        self.np_dtype = np_dtype_of(config)
        self.torch_dtype = torch.uint8 if self.np_dtype == np.uint8 else torch.int16
        self.num_layers = len(self.layer_map)
        self.device = torch.device(device)
        self.buf = torch.zeros((kv_slots, self.num_layers, self.top_k), dtype=self.torch_dtype, device=self.device)

    def capture(self, layer: int, ids: torch.Tensor, mem_index: torch.Tensor) -> None:
        """ids [T, k] int32 (the router's choice), mem_index [T] (KV slots of these tokens)."""
        j = self.layer_map.get(layer)
        if j is None or ids.shape[0] != mem_index.shape[0] or ids.shape[0] == 0:
            return
        if not ids.is_cuda:
            self.buf[mem_index.long(), j] = ids.to(self.torch_dtype)
            return
        from ..ops import _count
        from ..ops._native import check, kernels, ptr, stream

        assert ids.dtype == torch.int32 and ids.is_contiguous() and mem_index.dtype == torch.int32
        check(kernels().llb_route_capture(ptr(ids), ptr(mem_index), ctypes.c_int(ids.shape[0]),
                                          ctypes.c_int(self.top_k), ptr(self.buf), ctypes.c_int(self.buf.shape[0]),
                                          ctypes.c_int(self.num_layers), ctypes.c_int(j),
                                          ctypes.c_int(self.buf.element_size()), stream()), "route_capture")
        _count()

    def extract(self, slots: torch.Tensor) -> np.ndarray:
        """[n, moe layers, top_k] of the given KV slots (host array)."""
        rows = self.buf.index_select(0, slots.to(self.device).long())
        return rows.cpu().numpy()
