"""Messages that travel between the processes of a server (zmq pickles / the shm mailbox).

Reference: lightllm/server/core/objs/io_objs/group_req.py, lightllm/server/io_struct.py.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Optional


@dataclass
class GroupReqIndexes:
    """All sub-requests (n > 1) of one user request: slot indices into the shm request array."""

    group_req_id: int
    multimodal_params: Any
    shm_req_indexes: List[int]
    time_mark: float = 0.0


@dataclass
class GroupReqObjs:
    group_req_id: int
    multimodal_params: Any
    shm_req_objs: List[Any]
    time_mark: float = 0.0

    def to_group_req_index(self) -> GroupReqIndexes:
        return GroupReqIndexes(self.group_req_id, self.multimodal_params,
                               [r.index_in_shm_mem for r in self.shm_req_objs], self.time_mark)


@dataclass
class AbortedReqCmd:
    req_id: int


@dataclass
class StopStrMatchedReqCmd:
    req_id: int


@dataclass
class ProfilerCmd:
    cmd: str  # "start" | "stop"


@dataclass
class FlushCacheCmd:
    pass


@dataclass
class RLCmd:
    """RL control plane operation fanned out to every rank (pause handled in the HTTP layer)."""

    op: str
    payload: Any = None


@dataclass
class NewReqsCmd:
    """(req_id, shm_index, multimodal_params, dp_index) tuples of a newly scheduled batch."""

    reqs: List[tuple] = field(default_factory=list)
