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


def _weight_slots(m):
    """(owner, attribute, tensor) of every plain weight tensor of the model: layer tables first, then the
    embedding, the final norm and the head (which may be the embedding itself)."""
    for lw in m.layers:
        for k, t in list(lw.tensors().items()):
            if isinstance(t, torch.Tensor):
                yield lw, k, t
    for k in ("embed_w", "final_norm_w", "lm_head_w"):
        t = getattr(m, k, None)
        if isinstance(t, torch.Tensor):
            yield m, k, t


def release_memory_occupation(loop, tags=("kv_cache",)):
    """Frees the KV pool and / or the weights so that a co-located trainer can use the GPU.  Weights: with
    `--enable_weight_cpu_backup` they are copied to (pinned) host memory first and come back on resume; without,
    only their shapes are kept and resume hands out zeroed tensors that the trainer's next weight push fills.
    Reference: lightllm/common/basemodel/basemodel.py:100-116 (memory-saver regions, `enable_cpu_backup`)."""
    m = loop.model
    if loop.backend.has_work():
        raise RuntimeError("cannot release memory while requests are running")
    flush_cache(loop)
    m.flush_graphs()
    if "kv_cache" in tags and m.mem_manager.kv_buffer is not None:
        m._released_kv_shape = tuple(m.mem_manager.kv_buffer.shape)
        m.mem_manager.kv_buffer = None
    if "weights" in tags and getattr(m, "_weight_backup", None) is None:
        keep = bool(getattr(getattr(loop, "args", None), "enable_weight_cpu_backup", True))
        saved, slots = {}, []          # one entry per storage: tied tensors stay tied after resume
        for owner, k, t in _weight_slots(m):
            key = (t.data_ptr(), tuple(t.shape), t.dtype)
            if key not in saved:
                if keep:
                    host = torch.empty(t.shape, dtype=t.dtype, pin_memory=t.is_cuda)
                    host.copy_(t)
                    saved[key] = host
                else:
                    saved[key] = (tuple(t.shape), t.dtype)
            slots.append((owner, k, key))
        for owner, k, _ in slots:
            setattr(owner, k, None)
        m._weight_backup = (keep, saved, slots)
    if m.device.type == "cuda":
        torch.cuda.empty_cache()


def resume_memory_occupation(loop, tags=("kv_cache",)):
    m = loop.model
    if "kv_cache" in tags and m.mem_manager.kv_buffer is None:
        m.mem_manager.kv_buffer = torch.zeros(m._released_kv_shape, dtype=m.mem_manager.dtype, device=m.device)
    if "weights" in tags and getattr(m, "_weight_backup", None):
        keep, saved, slots = m._weight_backup
        live = {}
        for owner, k, key in slots:
            if key not in live:
                v = saved[key]
                live[key] = v.to(m.device, non_blocking=True) if keep else torch.zeros(v[0], dtype=v[1], device=m.device)
            setattr(owner, k, live[key])
        if m.device.type == "cuda":
            torch.cuda.synchronize()
        m._weight_backup = None


def update_weights_from_tensor(loop, named_tensors, weight_version=None, flush=True):
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
    if flush:
        flush_cache(loop)


_update_groups = {}


def init_weights_update_group(loop, master_address, master_port, rank_offset, world_size,
                              group_name="weight_update_group", backend="nccl"):
    """Joins the trainer's weight-update group as rank `rank_offset + global rank` (the trainer is rank 0 and hosts
    the store).  Blocks until every member is there."""
    from ..utils.rl_group import join_weight_update_group

    if not group_name:
        raise ValueError("group name cannot be empty")
    if group_name in _update_groups:
        raise ValueError(f"process group {group_name!r} already exists")
    if loop.model.device.type != "cuda":
        backend = "gloo"
    rank = int(rank_offset) + loop.ps.global_rank
    _update_groups[group_name] = join_weight_update_group(master_address, int(master_port), rank, int(world_size),
                                                          group_name, backend)


def destroy_weights_update_group(loop, group_name="weight_update_group"):
    pg = _update_groups.pop(group_name, None)
    if pg is None:
        raise ValueError(f"the group {group_name!r} does not exist")
    del pg


def update_weights_from_distributed(loop, names, dtypes, shapes, group_name="weight_update_group", flush=True,
                                    weight_version=None):
    """Receives the named tensors (full, unsharded, HF names) by broadcast from the trainer and loads them through
    the model's own loader, which takes this rank's slices."""
    from ..utils.rl_group import broadcast_from_trainer

    if group_name not in _update_groups:
        raise ValueError(f"group {group_name!r} unknown: call init_weights_update_group first")
    pg = _update_groups[group_name]
    dev = loop.model.device
    named = []
    for name, dtype, shape in zip(names, dtypes, shapes):
        dt = dtype if isinstance(dtype, torch.dtype) else getattr(torch, str(dtype).replace("torch.", ""))
        t = torch.empty(tuple(shape), dtype=dt, device=dev)
        broadcast_from_trainer(pg, t)
        named.append((name, t))
    update_weights_from_tensor(loop, named, weight_version, flush=flush)


def update_weights_from_ipc(loop, ipc_handle=None, use_shm=False, flush=True, weight_version=None):
    """Weights handed over by a trainer on the same host.  `ipc_handle` (a dict, or a dict of such per rank in the
    node) names either a POSIX shared-memory segment written with `utils.rl_group`-style manifests
    ({"shm_name", "manifest": [[name, dtype, shape, byte offset], ...]}, `use_shm`) or CUDA IPC handles
    ({"tensors": [[name, dtype, shape, base64 handle, byte offset], ...]}): the rank maps the memory, copies the
    tensors into its own weights and unmaps it again."""
    import base64
    import numpy as np

    h = ipc_handle
    if isinstance(h, dict) and not ({"shm_name", "tensors"} & set(h)):
        h = h.get(loop.ps.local_rank, h.get(str(loop.ps.local_rank)))
    if not isinstance(h, dict):
        raise ValueError("update_weights_from_ipc: no handle for this rank")
    dev = loop.model.device
    named = []
    if use_shm or "shm_name" in h:
        from multiprocessing import shared_memory

        shm = shared_memory.SharedMemory(name=h["shm_name"])
        try:
            for name, dtype, shape, off in h["manifest"]:
                dt = getattr(torch, str(dtype).replace("torch.", ""))
                n = int(np.prod(shape)) * torch.empty(0, dtype=dt).element_size()
                t = torch.frombuffer(shm.buf, dtype=torch.uint8, count=n, offset=int(off)).view(dt).view(*shape)
                named.append((name, t.to(dev).clone()))
                del t
        finally:
            shm.close()
    else:
        import ctypes

        from ..ops._native import check, kernels
        from ..parallel.symm import view_device_memory

        lib = kernels()
        for name, dtype, shape, handle_b64, off in h["tensors"]:
            dt = getattr(torch, str(dtype).replace("torch.", ""))
            n = int(np.prod(shape)) * torch.empty(0, dtype=dt).element_size()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(base64.b64decode(handle_b64))
            base = ctypes.c_void_p()
            check(lib.llb_ipc_open_handle(buf, ctypes.byref(base)), "ipc_open_handle")
            try:
                src = view_device_memory(base.value + int(off), n, dev).view(dt).view(*shape)
                named.append((name, src.clone()))
                torch.cuda.synchronize(dev)
            finally:
                lib.llb_ipc_close_handle(base)
    update_weights_from_tensor(loop, named, weight_version, flush=flush)


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
    elif op == "init_weights_update_group":
        init_weights_update_group(loop, payload["master_address"], payload["master_port"], payload.get("rank_offset", 1),
                                  payload["world_size"], payload.get("group_name", "weight_update_group"),
                                  payload.get("backend", "nccl"))
    elif op == "destroy_weights_update_group":
        destroy_weights_update_group(loop, payload.get("group_name", "weight_update_group"))
    elif op == "update_weights_from_distributed":
        update_weights_from_distributed(loop, payload["names"], payload["dtypes"], payload["shapes"],
                                        payload.get("group_name", "weight_update_group"),
                                        payload.get("flush_cache", True), payload.get("weight_version"))
    elif op == "update_weights_from_ipc":
        update_weights_from_ipc(loop, payload.get("ipc_handle"), payload.get("use_shm", False),
                                payload.get("flush_cache", True), payload.get("weight_version"))
    else:
        raise ValueError(f"unknown RL op {op}")
