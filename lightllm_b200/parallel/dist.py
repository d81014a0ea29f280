"""Rank bookkeeping and process groups.

Same vocabulary as the reference (lightllm/utils/dist_utils.py:7-44): ``--tp`` is the total
world size, ``--dp`` splits it into data-parallel attention replicas, each replica being a
tensor-parallel group of ``tp // dp`` ranks.  One process per GPU; torch.distributed (NCCL on
GPUs, gloo on CPU) carries the bootstrap and the baseline collectives, the fused kernels in
``parallel.fused`` ride on peer memory obtained through it.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class ParallelState:
    world_size: int = 1
    global_rank: int = 0
    dp_size: int = 1              # number of attention replicas
    tp_size: int = 1              # ranks inside one replica (= world // dp)
    dp_rank: int = 0              # which replica this rank belongs to
    tp_rank: int = 0              # rank inside the replica
    nnodes: int = 1
    node_rank: int = 0
    local_rank: int = 0           # rank inside the node (device index)
    backend: str = "none"
    device: torch.device = torch.device("cpu")
    tp_group: Optional[object] = None      # ranks of my replica
    world_group: Optional[object] = None
    node_group: Optional[object] = None
    dp_peer_group: Optional[object] = None  # same tp_rank across replicas
    cpu_group: Optional[object] = None      # gloo group over the world for host-side sync

    @property
    def is_first_rank(self) -> bool:
        return self.global_rank == 0

    @property
    def ep_size(self) -> int:
        return self.world_size


_STATE = ParallelState()


def state() -> ParallelState:
    return _STATE


def init_distributed(world_size: int = 1, rank: int = 0, dp: int = 1, nnodes: int = 1, node_rank: int = 0,
                     host: str = "127.0.0.1", port: int = 28765, backend: Optional[str] = None,
                     device: Optional[torch.device] = None, timeout_s: float = 1800.0,
                     config_server: Optional[tuple] = None) -> ParallelState:
    """Create the world group and the derived groups; a 1-element all-reduce warms the backend up
    (reference: lightllm/utils/dist_utils.py:130-161).

    `config_server` = (host, http port): `--use_config_server_to_init_nccl`.  The rendezvous store then lives in
    the config server (rank 0 asks it to start one on `port`, the other ranks wait until it is up) and every rank,
    rank 0 included, joins as a client, so a model world can be restarted without rank 0's port lingering
    (reference: lightllm/utils/dist_utils.py:293-318)."""
    global _STATE
    assert world_size % dp == 0, "--dp must divide --tp"
    per_node = world_size // nnodes
    local_rank = rank % per_node
    if device is None:
        device = torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu")
    if backend is None:
        backend = "nccl" if device.type == "cuda" else "gloo"
    st = ParallelState(world_size=world_size, global_rank=rank, dp_size=dp, tp_size=world_size // dp,
                       dp_rank=rank // (world_size // dp), tp_rank=rank % (world_size // dp), nnodes=nnodes,
                       node_rank=node_rank, local_rank=local_rank, backend=backend, device=device)
    if device.type == "cuda":
        torch.cuda.set_device(device)
    if world_size > 1:
        if not dist.is_initialized() and config_server is not None:
            _external_store(config_server, port, rank, world_size)
        if not dist.is_initialized():
            dist.init_process_group(backend, init_method=f"tcp://{host}:{port}", world_size=world_size, rank=rank,
                                    timeout=datetime.timedelta(seconds=timeout_s))
        st.world_group = dist.group.WORLD
        tp = st.tp_size
        # tensor-parallel group of each replica
        for r in range(dp):
            ranks = list(range(r * tp, (r + 1) * tp))
            g = dist.new_group(ranks) if tp > 1 and dp > 1 else None
            if r == st.dp_rank:
                st.tp_group = g if dp > 1 else (dist.group.WORLD if tp > 1 else None)
        # same tp_rank across replicas
        if dp > 1:
            for t in range(tp):
                ranks = [r * tp + t for r in range(dp)]
                g = dist.new_group(ranks)
                if t == st.tp_rank:
                    st.dp_peer_group = g
        if nnodes > 1:
            for n in range(nnodes):
                g = dist.new_group(list(range(n * per_node, (n + 1) * per_node)))
                if n == node_rank:
                    st.node_group = g
        else:
            st.node_group = dist.group.WORLD
        st.cpu_group = dist.new_group(list(range(world_size)), backend="gloo") if backend != "gloo" else dist.group.WORLD
        warm = torch.ones(1, device=device)
        dist.all_reduce(warm)
    _STATE = st
    return st


def init_from_env(dp: int = 1) -> ParallelState:
    """torchrun-style bootstrap (RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT / LOCAL_RANK)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    host = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", "28765"))
    return init_distributed(world, rank, dp=dp, host=host, port=port)


def _external_store(config_server, store_port: int, rank: int, world_size: int, wait_s: float = 180.0):
    """Asks the config server for a rendezvous store on `store_port` and makes this process join it as a client."""
    import json
    import time
    import urllib.error
    import urllib.request

    host, http_port = config_server
    url = f"http://{host}:{http_port}/start_tcp_store_server?tcp_store_port={store_port}&rank_id={rank}" \
          f"&world_size={world_size}"
    t0 = time.time()
    while True:
        try:
            with urllib.request.urlopen(url, timeout=30) as r:
                if r.status == 200 and json.loads(r.read()).get("status") == "ok":
                    break
        except (urllib.error.URLError, OSError):
            pass                      # rank 0 has not asked yet (503) or the server is still coming up
        if time.time() - t0 > wait_s:
            raise TimeoutError(f"the config server at {host}:{http_port} did not provide a store on port {store_port}")
        time.sleep(0.2)
    os.environ["TORCHELASTIC_USE_AGENT_STORE"] = "True"     # torch: every rank is a client of the tcp:// store


def destroy(hard_exit_on_hang: bool = False, wait_s: float = 20.0):
    """Tear the process groups down.  Objects that still hold captured collectives (CUDA graphs) should be
    released first (`LLM.close()`); if the tear-down does not return within `wait_s` and `hard_exit_on_hang` is
    set (benchmarks, tests: their work is done and printed), the process exits at once instead of hanging."""
    global _STATE
    if dist.is_initialized():
        import gc
        import threading

        gc.collect()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        t = threading.Thread(target=dist.destroy_process_group, daemon=True)
        t.start()
        t.join(wait_s)
        if t.is_alive():
            import sys

            print(f"[dist] destroy_process_group still running after {wait_s:.0f}s", file=sys.stderr, flush=True)
            if hard_exit_on_hang:
                sys.stdout.flush()
                os._exit(0)
    _STATE = ParallelState()


# ---- baseline collectives (short-circuit on size-1 groups, like the reference's free functions
#      in lightllm/distributed/communication_op.py:326-408) ----
def all_reduce(x, group=None, op=dist.ReduceOp.SUM):
    if group is None:
        return x
    dist.all_reduce(x, op=op, group=group)
    return x


def all_gather_into_tensor(out, x, group=None):
    if group is None:
        out.copy_(x)
        return out
    dist.all_gather_into_tensor(out, x, group=group)
    return out


def reduce_scatter_tensor(out, x, group=None):
    if group is None:
        out.copy_(x)
        return out
    if x.device.type == "cpu":  # gloo has no reduce_scatter: all-reduce then slice
        tmp = x.clone()
        dist.all_reduce(tmp, group=group)
        n = out.shape[0]
        r = dist.get_rank(group)
        out.copy_(tmp[r * n:(r + 1) * n])
        return out
    dist.reduce_scatter_tensor(out, x, group=group)
    return out


def broadcast(x, src=0, group=None):
    if group is None:
        return x
    dist.broadcast(x, src=src, group=group)
    return x
