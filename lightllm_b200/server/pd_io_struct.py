"""Objects exchanged between pd_master, prefill (P) nodes and decode (D) nodes.

Everything here is plain picklable data; websocket frames are `pickle.dumps((tag, payload))`.
Reference: lightllm/server/pd_io_struct.py (PD_Client_Obj, UpKVStatus, KVMoveTask, PDTransJoinInfo ...).
"""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class NodeRole(enum.Enum):
    P = "prefill"
    D = "decode"
    NORMAL = "normal"
    PD_MASTER = "pd_master"

    def is_P(self):
        return self is NodeRole.P

    def is_D(self):
        return self is NodeRole.D

    def is_P_or_D(self):
        return self in (NodeRole.P, NodeRole.D)


@dataclass
class NodeRunStatus:
    """Load numbers a node reports with every heartbeat (the same as its /token_load route)."""
    total_token_usage_rate: float = 0.0
    running_reqs: int = 0
    waiting_reqs: int = 0
    stamp: float = field(default_factory=time.time)


@dataclass
class PDClient:
    node_id: int
    client_ip_port: str
    mode: str  # "prefill" | "decode"
    start_args: Dict[str, Any]
    websocket: Any = None
    run_status: NodeRunStatus = field(default_factory=NodeRunStatus)
    dispatched_req_num: int = 0  # requests in flight that the master sent to this node
    dispatched_prompt_chars: int = 0
    last_heartbeat: float = field(default_factory=time.time)

    def __post_init__(self):
        if self.mode not in ("prefill", "decode"):
            raise ValueError(f"mode must be prefill or decode, got {self.mode}")

    @property
    def kv_endpoint(self):
        """(ip, port) of the node's KV-transfer rendezvous store."""
        ip = self.client_ip_port.rsplit(":", 1)[0]
        return ip, int(self.start_args.get("pd_kv_port") or 0)

    def to_wire(self) -> dict:
        return {"node_id": self.node_id, "client_ip_port": self.client_ip_port, "mode": self.mode,
                "kv_endpoint": self.kv_endpoint, "tp": self.start_args.get("tp", 1),
                "dp": self.start_args.get("dp", 1)}


@dataclass
class PDMasterInfo:
    """What a pd_master leaves at the config server: prefill / decode nodes connect to `host_ip_port`."""
    node_id: int
    host_ip_port: str


@dataclass
class PDRegister:
    node_id: int
    client_ip_port: str
    mode: str
    start_args: Dict[str, Any]


@dataclass
class PDHeartbeat:
    node_id: int
    run_status: NodeRunStatus


@dataclass
class PDRequest:
    """master -> node.  For the D node `prompt` holds token ids (prompt + first token) and
    `first_token` the (id, logprob) that P produced, so that decode continues the same sequence."""
    group_req_id: int
    prompt: Any
    sampling_params: Dict[str, Any]
    multimodal_params: Optional[dict] = None
    peer: Optional[dict] = None  # the other node of the pair (PDClient.to_wire())
    first_token: Optional[tuple] = None


@dataclass
class PDToken:
    """node -> master: one generated token of a request."""
    group_req_id: int
    sub_req_id: int
    text: str
    metadata: Dict[str, Any]
    finish_status: int


@dataclass
class PDPromptIds:
    """P node -> master: the tokenised prompt (the master hands it to D with the first token)."""
    group_req_id: int
    prompt_ids: List[int]


@dataclass
class UpKVStatus:
    """D node -> master on /kv_move_status: the KV of `group_req_id` has fully arrived (or failed)."""
    group_req_id: int
    dp_index: int = 0
    ok: bool = True
    type: str = "kv_move_ok"


@dataclass
class KVMoveTask:
    """One staged page of a request's KV on its way P -> D.  `token_slots` are pool slots on the sender,
    `page_index` counts pages of the request, `last` marks the final page (it carries the first token)."""
    group_req_id: int
    page_index: int
    num_tokens: int
    token_slots: Any = None
    last: bool = False
    first_token: Optional[tuple] = None
    created: float = field(default_factory=time.time)

    def expired(self, timeout_s: float = 182.0) -> bool:
        return time.time() - self.created > timeout_s
