"""Keeps the routers of a multi-node tensor-parallel deployment (`--nnodes` > 1, `--dp` 1) identical.

Every node runs its own router in front of its share of the model ranks, and all ranks of the one replica must
see the same requests join and leave on the same step.  Node 0 is the master: requests reach the other nodes by
forwarding (same group request id everywhere), but not at the same instant, and only node 0 sees the client
connections.  So, over a host-side (gloo) group of the routers:

  * every node reports the ids waiting in its queue and whether its mailbox to the model ranks is free;
  * the master, if every mailbox is free, runs its Past-Future estimate over the requests that have arrived on ALL
    nodes (in its own arrival order) and broadcasts its plan: the group ids it admits, the other commands of this
    round (aborts, stop-string hits, profiler / cache / weight-update / exit commands, which only node 0 learns
    of) and the ids of waiting requests it dropped because their client went away;
  * every node takes exactly the admitted requests from its queue, in that order, and writes the same message to
    its ranks.  The ranks agree on the mailbox generation across nodes, so message k must be the same everywhere:
    that is why nothing node-local (its own view of finished or stopped requests) enters a message.

One all-gather and one broadcast of small python objects per scheduling round.
Reference: lightllm/server/router/multinode_tp_helper.py:1-219 (barrier, schedule as master / slave, two-phase abort).
"""
from __future__ import annotations

from typing import List, Optional, Set, Tuple

import torch.distributed as dist


class MultiNodeRouterSync:
    def __init__(self, group, node_rank: int, nnodes: int):
        self.group, self.node_rank, self.nnodes = group, node_rank, nnodes

    @property
    def is_master(self) -> bool:
        return self.node_rank == 0

    def gather(self, waiting_ids: List[int], mailbox_free: bool) -> Tuple[bool, Set[int]]:
        """(every node's mailbox is free, ids that wait on every node)."""
        views: List[Optional[tuple]] = [None] * self.nnodes
        dist.all_gather_object(views, (bool(mailbox_free), list(waiting_ids)), group=self.group)
        common = set(views[0][1])
        for _, ids in views[1:]:
            common &= set(ids)
        return all(v[0] for v in views), common

    def broadcast(self, plan):
        """The master's plan of this round for everybody (`plan` is ignored on the other nodes)."""
        box = [plan if self.is_master else None]
        src = dist.get_global_rank(self.group, 0) if self.group is not None else 0
        dist.broadcast_object_list(box, src=src, group=self.group)
        return box[0]
