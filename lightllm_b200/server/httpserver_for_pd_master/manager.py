"""pd_master front-end: keeps the registry of prefill (P) and decode (D) nodes, picks a pair per request,
drives the request through the pair and relays the token stream to the client.  No GPU in this process.

Per request:  master --PDRequest(peer=D)--> P;  P prefills, pushes the KV pages to D and uploads the tokenised
prompt and the first token;  D reports on /kv_move_status when all pages arrived;  master then sends
PDRequest(prompt ids + first token) to D, which decodes the rest and uploads tokens;  master yields them with the
same `(sub_req_id, text, metadata, FinishStatus)` contract as the single-node manager.

Topology (--pd_master_mode): `elastic` serves as soon as one P and one D are registered and nodes may come and
go; `<x>p<y>d` refuses requests until exactly that many of each have registered.
Reference: lightllm/server/httpserver_for_pd_master/manager.py, register_loop.py.
"""
from __future__ import annotations

import asyncio
import os
import pickle
import re
import time
from typing import Dict, List, Optional

from ...utils.errors import ServerBusyError
from ..core.objs.req import FinishStatus
from ..core.objs.sampling_params import SamplingParams
from ..pd_io_struct import PDClient, PDHeartbeat, PDPromptIds, PDRegister, PDRequest, PDToken, UpKVStatus
from ..req_id_generator import MAX_BEST_OF
from .selector import create_selector

HEARTBEAT_TIMEOUT_S = 90.0
FIRST_TOKEN_TIMEOUT_S = 600.0
KV_MOVE_TIMEOUT_S = 182.0


def split_block_tokens() -> int:
    try:
        return max(1, int(os.environ.get("LLB_PD_SPLIT_MAX_NEW_TOKENS", os.environ.get("LIGHTLLM_PD_SPLIT_MAX_NEW_TOKENS", "2048"))))
    except ValueError:
        return 2048


def split_max_new_tokens(max_new_tokens: int) -> List[int]:
    """Budgets of the blocks a request is served in: full blocks, then the rest."""
    b = split_block_tokens()
    full, rest = divmod(max(int(max_new_tokens), 0), b)
    return ([b] * full + ([rest] if rest else [])) or [int(max_new_tokens)]


class _ReqState:
    def __init__(self, group_req_id, p: PDClient, d: PDClient, prompt_chars: int):
        self.group_req_id, self.p, self.d, self.prompt_chars = group_req_id, p, d, prompt_chars
        self.tokens: asyncio.Queue = asyncio.Queue()
        self.prompt_ids: Optional[List[int]] = None
        self.kv_done = asyncio.Event()
        self.kv_ok = False


class HttpServerManagerForPDMaster:
    def __init__(self, args, metric_client=None):
        self.args = args
        self.metric_client = metric_client
        self.nodes: Dict[int, PDClient] = {}
        self.selector = create_selector(args.select_p_d_node_strategy)
        self.reqs: Dict[int, _ReqState] = {}
        self.alias: Dict[int, int] = {}             # a client request's id -> the id of the block it is in
        self.block_prompt_ids: Dict[int, List[int]] = {}
        self._next_id = MAX_BEST_OF
        self._id_end = 0                            # end of the id range drawn from the config server
        self.paused = False
        self.tokenizer = None
        m = re.fullmatch(r"(\d+)p(\d+)d", args.pd_master_mode or "elastic")
        self.fixed_topology = (int(m.group(1)), int(m.group(2))) if m else None
        if not m and (args.pd_master_mode or "elastic") != "elastic":
            raise ValueError("--pd_master_mode is 'elastic' or '<P>p<D>d'")

    # ---------------------------------------------------------------- ids
    async def _take_id(self) -> int:
        """The next request id.  Several pd_masters behind one config server draw disjoint ranges from it
        (`/allocate_global_unique_id_range`), so that ids stay unique on the nodes they share."""
        host, port = getattr(self.args, "config_server_host", None), getattr(self.args, "config_server_port", None)
        if host and port:
            if self._next_id + MAX_BEST_OF > self._id_end:
                import requests

                def fetch():
                    r = requests.get(f"http://{host}:{port}/allocate_global_unique_id_range", timeout=10)
                    r.raise_for_status()
                    return r.json()

                got = await asyncio.to_thread(fetch)
                first = -(-int(got["start_id"]) // MAX_BEST_OF) * MAX_BEST_OF
                self._next_id, self._id_end = max(first, MAX_BEST_OF), int(got["end_id"])
        gid = self._next_id
        self._next_id += MAX_BEST_OF
        return gid

    async def keep_registered_at_config_server(self, beat_s: float = 10.0):
        """Holds the websocket that lists this master at the config server (prefill / decode nodes find the masters
        there); opens it again when it breaks.  Reference: httpserver_for_pd_master/register_loop.py."""
        import websockets

        from ..pd_io_struct import PDMasterInfo

        a = self.args
        info = PDMasterInfo(os.getpid(), f"{a.host}:{a.port}")
        while True:
            try:
                async with websockets.connect(f"ws://{a.config_server_host}:{a.config_server_port}/pd_master_register",
                                              max_size=None) as ws:
                    await ws.send(pickle.dumps(info))
                    while True:
                        await ws.send("beat")
                        await asyncio.sleep(beat_s)
            except asyncio.CancelledError:
                raise
            except Exception as e:  # noqa: BLE001
                print(f"[pd_master] config server not reachable ({type(e).__name__}: {e}); retrying", flush=True)
                await asyncio.sleep(3.0)

    # ---------------------------------------------------------------- registry
    def _refresh(self):
        ps = [n for n in self.nodes.values() if n.mode == "prefill"]
        ds = [n for n in self.nodes.values() if n.mode == "decode"]
        self.selector.update_nodes(ps, ds)
        return ps, ds

    async def register_pd(self, reg: PDRegister, websocket) -> PDClient:
        node = PDClient(reg.node_id, reg.client_ip_port, reg.mode, reg.start_args, websocket)
        self.nodes[reg.node_id] = node
        self._refresh()
        return node

    async def remove_pd(self, node_id: int):
        node = self.nodes.pop(node_id, None)
        if node is None:
            return
        self.selector.forget_node(node)
        self._refresh()
        for st in list(self.reqs.values()):  # requests on the lost node end with an error
            if st.p is node or st.d is node:
                st.kv_ok = False
                st.kv_done.set()
                await st.tokens.put(PDToken(st.group_req_id, st.group_req_id, "", {"error": "pd node lost"},
                                            FinishStatus.FINISHED_ERROR))

    def update_node_status(self, hb: PDHeartbeat):
        node = self.nodes.get(hb.node_id)
        if node is not None:
            node.run_status, node.last_heartbeat = hb.run_status, time.time()

    async def drop_silent_nodes(self, now=None):
        now = now or time.time()
        for nid, n in list(self.nodes.items()):
            if now - n.last_heartbeat > HEARTBEAT_TIMEOUT_S:
                await self.remove_pd(nid)

    def topology_ready(self) -> bool:
        ps, ds = self._refresh()
        if self.fixed_topology:
            return (len(ps), len(ds)) == self.fixed_topology
        return bool(ps) and bool(ds)

    # ---------------------------------------------------------------- node -> master
    async def on_node_message(self, obj):
        if isinstance(obj, PDHeartbeat):
            self.update_node_status(obj)
        elif isinstance(obj, PDPromptIds):
            st = self.reqs.get(obj.group_req_id)
            if st is not None:
                st.prompt_ids = obj.prompt_ids
        elif isinstance(obj, PDToken):
            st = self.reqs.get(obj.group_req_id)
            if st is not None:
                await st.tokens.put(obj)
        elif isinstance(obj, UpKVStatus):
            await self.update_kv_move_status(obj)

    async def update_kv_move_status(self, up: UpKVStatus):
        st = self.reqs.get(up.group_req_id)
        if st is not None:
            st.kv_ok = up.ok
            st.kv_done.set()

    # ---------------------------------------------------------------- generate
    @staticmethod
    async def _send(node: PDClient, obj):
        await node.websocket.send_bytes(pickle.dumps(obj))

    def tokens(self, prompt, multimodal_params=None, samping_params=None, kwargs=None) -> int:
        raise ValueError("the pd_master has no tokenizer; ask a prefill node")

    async def generate(self, prompt, sampling_params: SamplingParams, multimodal_params=None, request=None,
                       is_health_req: bool = False):
        """One client request.  A long `max_new_tokens` is served in blocks of `split_block_tokens()`: decode nodes
        schedule conservatively (they reserve room for every token a request may still produce), so one request
        that asks for a huge budget would hold a node's pool on its own; each block is a request of its own on the
        same pair of nodes whose prompt is the original prompt plus everything generated so far (the prefill
        node finds all but the last block's tokens in its prefix cache).  Most requests end inside their first
        block.  Reference: httpserver_for_pd_master/manager.py:204-268, 662-668."""
        if self.paused and not is_health_req:
            raise ServerBusyError("generation is paused")
        if not self.topology_ready():
            raise ServerBusyError("no complete prefill/decode topology is registered")
        if sampling_params.n != 1:
            raise ValueError("pd_master mode serves n == best_of == 1")
        origin = await self._take_id()
        p, d = self.selector.select_p_d_node(prompt, sampling_params, multimodal_params)
        sp = sampling_params.to_dict()
        total = int(sp["max_new_tokens"])
        has_media = bool(multimodal_params) and any((multimodal_params or {}).get(k) for k in ("images", "audios")) \
            if isinstance(multimodal_params, dict) else bool(multimodal_params)
        blocks = [total] if has_media else split_max_new_tokens(total)   # a picture's ids cannot be sent back as text
        start = time.time()
        produced, history, first_meta, prompt_ids = 0, [], None, None
        block_prompt = prompt
        try:
            for bi, budget in enumerate(blocks):
                last = bi == len(blocks) - 1
                gid = origin if bi == 0 else await self._take_id()
                self.alias[origin] = gid
                sp_b = dict(sp)
                sp_b["max_new_tokens"] = budget
                sp_b["min_new_tokens"] = max(1, int(sp.get("min_new_tokens", 1)) - produced)
                ended = False
                block = self._run_block(gid, p, d, block_prompt, sp_b, multimodal_params, request, start)
                async for _, text, meta, fs in block:
                    if first_meta is None:
                        first_meta = dict(meta)
                        prompt_ids = self.block_prompt_ids.pop(gid, None)
                    if "id" in meta:
                        history.append(int(meta["id"]))
                    if bi > 0:      # what the client sees describes the whole request, not the block
                        meta = dict(meta)
                        if "count_output_tokens" in meta:
                            meta["count_output_tokens"] += produced
                        for k in ("prompt_tokens", "prompt_cache_len"):
                            if k in first_meta:
                                meta[k] = first_meta[k]
                    if fs.is_finished() and fs.get_finish_reason() == "length" and not last and "error" not in meta:
                        fs = FinishStatus()              # the block's budget, not the request's
                    elif fs.is_finished():
                        ended = True
                    try:
                        yield origin, text, meta, fs
                    except GeneratorExit:
                        await block.aclose()         # the client went away: the block's bookkeeping ends with it
                        raise
                    if ended:
                        await block.aclose()
                        return
                produced += budget
                if prompt_ids is None or len(history) < produced:
                    return                                # the stream broke off without an end mark
                block_prompt = list(prompt_ids) + history
        finally:
            self.alias.pop(origin, None)

    async def _run_block(self, gid, p, d, prompt, sp: dict, multimodal_params, request, start):
        chars = len(prompt)
        st = self.reqs[gid] = _ReqState(gid, p, d, chars)
        for n in (p, d):
            n.dispatched_req_num += 1
        p.dispatched_prompt_chars += chars
        sp = dict(sp)
        sp["group_request_id"] = gid
        try:
            await self._send(p, PDRequest(gid, prompt, sp, multimodal_params, peer=d.to_wire()))
            first: PDToken = await asyncio.wait_for(st.tokens.get(), FIRST_TOKEN_TIMEOUT_S)
            fs = FinishStatus(first.finish_status)
            meta = dict(first.metadata)
            meta["first_token_cost_ms"] = (time.time() - start) * 1e3
            if "prompt_cache_len" in meta and meta.get("prompt_tokens"):
                self.selector.record_prompt_cache_hit_rate(meta["prompt_cache_len"] / meta["prompt_tokens"])
            if st.prompt_ids is not None:
                self.block_prompt_ids[gid] = st.prompt_ids
            yield first.sub_req_id, first.text, meta, fs
            if fs.is_finished():
                return
            try:
                await asyncio.wait_for(st.kv_done.wait(), KV_MOVE_TIMEOUT_S)
            except asyncio.TimeoutError:
                st.kv_ok = False
            if not st.kv_ok or st.prompt_ids is None:
                yield first.sub_req_id, "", {"error": "kv transfer failed"}, FinishStatus(FinishStatus.FINISHED_ERROR)
                return
            sp_d = dict(sp)
            sp_d["max_new_tokens"] = max(1, int(sp["max_new_tokens"]) - 1)
            sp_d["min_new_tokens"] = max(1, int(sp.get("min_new_tokens", 1)) - 1)
            await self._send(d, PDRequest(gid, st.prompt_ids + [meta["id"]], sp_d, multimodal_params, peer=p.to_wire(),
                                          first_token=(meta["id"], meta.get("logprob", 0.0))))
            while True:
                tok: PDToken = await asyncio.wait_for(st.tokens.get(), FIRST_TOKEN_TIMEOUT_S)
                if request is not None and await request.is_disconnected():
                    await self.abort(gid)
                    raise asyncio.CancelledError(f"client disconnected, req {gid} aborted")
                m = dict(tok.metadata)
                m.setdefault("prompt_tokens", meta.get("prompt_tokens", len(st.prompt_ids)))
                if "count_output_tokens" in m:
                    m["count_output_tokens"] += 1  # D counts from its own first step
                fs = FinishStatus(tok.finish_status)
                yield tok.sub_req_id, tok.text, m, fs
                if fs.is_finished():
                    return
        finally:
            self.reqs.pop(gid, None)
            self.block_prompt_ids.pop(gid, None)
            for n in (p, d):
                n.dispatched_req_num = max(0, n.dispatched_req_num - 1)
            p.dispatched_prompt_chars = max(0, p.dispatched_prompt_chars - chars)

    async def abort(self, group_req_id: int) -> bool:
        """`group_req_id` is the id the client's stream carries; the nodes know the running block's id."""
        gid = self.alias.get(group_req_id, group_req_id)
        st = self.reqs.get(gid)
        if st is None:
            return False
        for n in (st.p, st.d):
            try:
                await self._send(n, ("ABORT", gid))
            except Exception:
                pass
        return True

    async def abort_all(self):
        for gid in list(self.reqs):
            await self.abort(gid)

    async def handle_loop(self):
        while True:
            await asyncio.sleep(10)
            await self.drop_silent_nodes()

    async def flush_cache(self):
        for n in self.nodes.values():
            await self._send(n, ("FLUSH_CACHE", None))

    async def rl_op(self, op, payload=None):
        for n in self.nodes.values():
            await self._send(n, ("RL", (op, payload)))

    async def profiler_cmd(self, what):
        for n in self.nodes.values():
            await self._send(n, ("PROFILER", what))
