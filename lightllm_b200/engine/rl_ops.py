"""RL control-plane operations executed on every model rank: flush the prefix cache, release /
resume GPU memory, live weight updates from a trainer.
Reference: lightllm/server/router/model_infer/mode_backend/rl_backend_ops.py, lightllm/utils/rl/*.
"""
from __future__ import annotations

import torch


def flush_cache(loop):
    b = loop.backend
    if b.has_work():
        return False
    if b.radix_cache is not None:
        b.radix_cache.clear_tree_nodes()
    return True


def release_memory_occupation(loop, tags=("kv_cache",)):
    """Frees the KV pool (and optionally weights to a host backup) so a co-located trainer can use the GPU."""
    m = loop.model
    if loop.backend.has_work():
        raise RuntimeError("cannot release memory while requests are running")
    flush_cache(loop)
    m.flush_graphs()
    if "kv_cache" in tags:
        m._released_kv_shape = tuple(m.mem_manager.kv_buffer.shape)
        m.mem_manager.kv_buffer = None
    if "weights" in tags:
        m._weight_backup = {}
        for i, lw in enumerate(m.layers):
            for k, t in list(lw.tensors().items()):
                if isinstance(t, torch.Tensor):
                    m._weight_backup[(i, k)] = t.cpu()
                    setattr(lw, k, None)
    if m.device.type == "cuda":
        torch.cuda.empty_cache()


def resume_memory_occupation(loop, tags=("kv_cache",)):
    m = loop.model
    if "kv_cache" in tags and m.mem_manager.kv_buffer is None:
        m.mem_manager.kv_buffer = torch.zeros(m._released_kv_shape, dtype=m.mem_manager.dtype, device=m.device)
    if "weights" in tags and getattr(m, "_weight_backup", None):
        for (i, k), t in m._weight_backup.items():
            setattr(m.layers[i], k, t.to(m.device))
        m._weight_backup = None


def update_weights_from_tensor(loop, named_tensors, weight_version=None):
    """named_tensors: iterable of (HF name, full tensor). Re-slices through the model's own loader."""
    from ..models.weights import WeightSource

    m = loop.model

    class _Patch(WeightSource):
        def __init__(self, base, patch):
            self.base, self.patch = base, dict(patch)

        def has(self, n):
            return n in self.patch or self.base.has(n)

        def shape(self, n):
            return tuple(self.patch[n].shape) if n in self.patch else self.base.shape(n)

        def names(self):
            return self.base.names()

        def get(self, n, dim=None, start=0, end=None):
            if n in self.patch:
                t = self.patch[n]
                if dim is not None:
                    t = t.narrow(dim, start, (end if end is not None else t.shape[dim]) - start)
                return t
            return self.base.get(n, dim, start, end)

    m.flush_graphs()
    m.weight_source = _Patch(m.weight_source, named_tensors)
    m._load_weights(m.weight_source)
    if weight_version is not None:
        m.weight_version = weight_version
    flush_cache(loop)


def handle_rl_cmd(loop, cmd):
    op, payload = cmd.op, cmd.payload or {}
    if op == "flush_cache":
        flush_cache(loop)
    elif op == "release_memory_occupation":
        release_memory_occupation(loop, tuple(payload.get("tags", ("kv_cache",))))
    elif op == "resume_memory_occupation":
        resume_memory_occupation(loop, tuple(payload.get("tags", ("kv_cache",))))
    elif op == "update_weights_from_tensor":
        update_weights_from_tensor(loop, payload["named_tensors"], payload.get("weight_version"))
    elif op == "update_weights_from_disk":
        from ..models.weights import SafetensorsSource

        loop.model.flush_graphs()
        loop.model.weight_source = SafetensorsSource(payload["model_dir"])
        loop.model._load_weights(loop.model.weight_source)
        loop.model.weight_version = payload.get("weight_version", loop.model.weight_version)
        flush_cache(loop)
    else:
        raise ValueError(f"unknown RL op {op}")
