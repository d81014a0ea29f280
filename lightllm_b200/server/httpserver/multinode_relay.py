"""Request relay between the HTTP servers of a multi-node tensor-parallel deployment (`--nnodes` > 1, `--dp` 1).

Clients talk to node 0 only.  Its HTTP server tokenises a request, gives it a group id and relays (id, token ids,
sampling parameters, multimodal parameters) to the HTTP server of every other node, which queues the same request
under the same id with its own router; the routers then admit it on the same step (`router/multinode_sync.py`).
The other nodes produce the same tokens and simply drop them.

Wire: node 0 binds a ZeroMQ ROUTER socket on `--multinode_httpmanager_port`; every other node connects a DEALER
to `--nccl_host` and says hello with its node rank; node 0 serves requests once all have said hello, so nothing is
relayed into the void.  Messages are signed (`LLB_RELAY_AUTHKEY`, else a key derived from `--nccl_host` and the
port) and checked before they are unpickled.  Reference: lightllm/server/httpserver/manager.py:91-104, 201-260 (multinode_req_manager,
loop_for_request, transfer of (prompt, sampling_params, multimodal_params) to the slave nodes).
"""
from __future__ import annotations

import asyncio
import time
from typing import Dict

import zmq
import zmq.asyncio

from ...utils.log_utils import init_logger
from ...utils.signed_msg import derive_key, seal, unseal

logger = init_logger(__name__)


def relay_key(args) -> bytes:
    return derive_key("LLB_RELAY_AUTHKEY", f"{getattr(args, 'nccl_host', None)}:"
                                           f"{getattr(args, 'multinode_httpmanager_port', None)}")


def enabled(args) -> bool:
    return int(getattr(args, "nnodes", 1)) > 1 and int(getattr(args, "dp", 1)) == 1


class RelayMaster:
    def __init__(self, port: int, n_peers: int, host: str = "0.0.0.0", key: bytes = b""):
        self.key = key or derive_key("LLB_RELAY_AUTHKEY", str(port))
        self.sock = zmq.asyncio.Context.instance().socket(zmq.ROUTER)
        self.sock.bind(f"tcp://{host}:{port}")
        self.n_peers = n_peers
        self.peers: Dict[int, bytes] = {}

    async def wait_peers(self, timeout_s: float = 600.0):
        t0 = time.time()
        while len(self.peers) < self.n_peers:
            left = timeout_s - (time.time() - t0)
            if left <= 0 or not await self.sock.poll(int(min(left, 1.0) * 1000)):
                if left <= 0:
                    raise TimeoutError(f"{self.n_peers - len(self.peers)} node(s) never connected to the request relay")
                continue
            ident, *frames = await self.sock.recv_multipart()
            try:
                msg = unseal(self.key, frames)
            except PermissionError as e:
                logger.warning(f"dropped a message: {e}")
                continue
            if msg[0] == "hello":
                self.peers[int(msg[1])] = ident
                await self.sock.send_multipart([ident] + seal(self.key, ("welcome",)))

    async def relay(self, group_req_id: int, prompt_ids, sampling_params, multimodal_params):
        frames = seal(self.key, ("req", group_req_id, list(prompt_ids), bytes(sampling_params), multimodal_params))
        for ident in self.peers.values():
            await self.sock.send_multipart([ident] + frames)

    def close(self):
        self.sock.close(linger=0)


class RelayFollower:
    def __init__(self, master_host: str, port: int, node_rank: int, key: bytes = b""):
        self.key = key or derive_key("LLB_RELAY_AUTHKEY", str(port))
        self.sock = zmq.asyncio.Context.instance().socket(zmq.DEALER)
        self.sock.connect(f"tcp://{master_host}:{port}")
        self.node_rank = node_rank
        self.tasks = set()

    async def hello(self, timeout_s: float = 600.0):
        t0 = time.time()
        while time.time() - t0 < timeout_s:       # node 0 may come up later than this node
            await self.sock.send_multipart(seal(self.key, ("hello", self.node_rank)))
            if await self.sock.poll(1000):
                assert unseal(self.key, await self.sock.recv_multipart())[0] == "welcome"
                return
        raise TimeoutError("node 0's request relay did not answer")

    async def follow(self, manager):
        """Queues every relayed request with this node's router and drains its output."""
        from ..core.objs.sampling_params import SamplingParams

        async def drain(gid, prompt_ids, sp, mm):
            try:
                async for _ in manager.generate(prompt_ids, sp, mm, group_req_id=gid):
                    pass
            except Exception as e:        # a request that fails here fails on node 0 for the same reason
                logger.warning(f"node {self.node_rank}: request {gid} ended with {type(e).__name__}: {e}")

        while True:
            try:
                msg = unseal(self.key, await self.sock.recv_multipart())
            except PermissionError as e:
                logger.warning(f"node {self.node_rank}: dropped a message: {e}")
                continue
            if msg[0] != "req":
                continue
            _, gid, prompt_ids, sp_bytes, mm = msg
            t = asyncio.create_task(drain(gid, prompt_ids, SamplingParams.from_buffer_copy(sp_bytes), mm))
            self.tasks.add(t)
            t.add_done_callback(self.tasks.discard)

    def close(self):
        self.sock.close(linger=0)
