"""Process group between a trainer and the model ranks of a running server, used to push new weights
(`/init_weights_update_group`, `/update_weights_from_distributed`).

The group is separate from the server's own groups: rank 0 is the trainer and hosts the rendezvous store at
`master_address:master_port`, the model ranks take `rank_offset + their global rank`.  A trainer joins with

    pg = join_weight_update_group(master_address, master_port, rank=0, world_size=1 + n_model_ranks)
    ...  POST /update_weights_from_distributed {"names": [...], "dtypes": [...], "shapes": [...]}  (do not wait)
    for t in tensors: broadcast_from_trainer(pg, t)

Reference: lightllm/utils/rl/ (init_custom_process_group), lightllm/server/router/model_infer/mode_backend/
rl_backend_ops.py:92-175.
"""
from __future__ import annotations

import datetime

import torch
import torch.distributed as dist


class WeightUpdateGroup:
    """The process group plus the store it was built on (which has to stay alive as long as the group)."""

    def __init__(self, pg, store, rank: int, world_size: int):
        self.pg, self.store, self.rank, self.world_size = pg, store, rank, world_size


def join_weight_update_group(master_address: str, master_port: int, rank: int, world_size: int,
                             group_name: str = "weight_update_group", backend: str = "nccl",
                             timeout_s: float = 300.0):
    """Blocks until all `world_size` members have joined.  `backend`: "nccl" (CUDA tensors) or "gloo"."""
    td = datetime.timedelta(seconds=timeout_s)
    store = dist.TCPStore(master_address, int(master_port), world_size, rank == 0, timeout=td,
                          wait_for_workers=False)
    store = dist.PrefixStore(group_name, store)
    if backend == "nccl":
        opts = dist.ProcessGroupNCCL.Options()
        opts._timeout = td
        pg = dist.ProcessGroupNCCL(store, rank, world_size, opts)
    elif backend == "gloo":
        pg = dist.ProcessGroupGloo(store, rank, world_size, td)
    else:
        raise ValueError(f"weight update group backend {backend!r}: use nccl or gloo")
    barrier_tensor = torch.zeros(1, device="cuda" if backend == "nccl" else "cpu")
    pg.allreduce([barrier_tensor]).wait()
    return WeightUpdateGroup(pg, store, rank, world_size)


def broadcast_from_trainer(group: WeightUpdateGroup, tensor: torch.Tensor):
    """In-place broadcast of `tensor` from rank 0 (the trainer) to every member."""
    opts = dist.BroadcastOptions()
    opts.rootRank = 0
    opts.rootTensor = 0
    group.pg.broadcast([tensor], opts).wait()
    return tensor
