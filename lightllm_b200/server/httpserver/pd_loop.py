"""P/D node side of the PD control plane: one task per pd_master keeps a websocket to `/pd_register`
open, registers, heartbeats every 30 s with the node's load, runs every PDRequest through the local
`generate()` and uploads the tokenised prompt and each token.  A lost connection is retried every 10 s
(elastic topology).  Reference: lightllm/server/httpserver/pd_loop.py.
"""
from __future__ import annotations

import asyncio
import os
import pickle
import traceback

from ..core.objs.sampling_params import SamplingParams
from ..pd_io_struct import NodeRunStatus, PDHeartbeat, PDPromptIds, PDRegister, PDRequest, PDToken, UpKVStatus

def ws_max_size():
    """Largest websocket message in bytes; unlimited unless LIGHTLLM_WEBSOCKET_MAX_SIZE says otherwise."""
    v = os.environ.get("LIGHTLLM_WEBSOCKET_MAX_SIZE")
    return int(v) if v else None


HEARTBEAT_S = 30.0
RETRY_S = 10.0


def node_id_of(args) -> int:
    return int(args.pd_node_id) if getattr(args, "pd_node_id", None) not in (None, -1) else \
        (hash((args.host, args.port)) & 0x7FFFFFFF)


def _run_status(g) -> NodeRunStatus:
    try:
        load = g.token_load
        cur = max(load.get_current_load(i) for i in range(load.dp))
    except Exception:
        cur = 0.0
    return NodeRunStatus(total_token_usage_rate=float(cur), running_reqs=len(g.httpserver_manager.req_id_to_out_inf))


async def serve_request(g, req: PDRequest, send):
    """Run one master request on this node and upload its stream."""
    mgr = g.httpserver_manager
    try:
        sp_kw = dict(req.sampling_params)
        sp_kw.pop("group_request_id", None)
        sp_kw.pop("suggested_dp_index", None)
        sp = SamplingParams().init(tokenizer=mgr.tokenizer, **sp_kw)
        sp.pd_master_node_id.set(int(req.peer["node_id"]) if req.peer else 0)
        mode = g.args.run_mode
        if mode == "decode" and int(getattr(g.args, "dp", 1) or 1) > 1:
            # the prefill node sent the KV to this replica (engine/mode_backends.py: decode_replica_of)
            from ...engine.mode_backends import decode_replica_of

            sp.suggested_dp_index = decode_replica_of(req.group_req_id, int(g.args.dp))
        if mode == "prefill":
            sp.max_new_tokens = 1  # P emits exactly the first token; the sequence continues on D
        pd_info = {"group_req_id": req.group_req_id, "peer": req.peer, "first_token": req.first_token}
        sent_ids = False
        async for sub_id, text, meta, fs in mgr.generate(req.prompt, sp, req.multimodal_params, None, pd_info=pd_info):
            if mode == "prefill" and not sent_ids:
                sent_ids = True
                await send(PDPromptIds(req.group_req_id, list(meta.pop("prompt_ids", []))))
            status = fs.get_status()
            if mode == "prefill" and fs.is_finished() and fs.get_finish_reason() == "length" and \
                    int(req.sampling_params.get("max_new_tokens", 1)) > 1:
                status = 0  # the length stop is this node's one-token cap, not the request's
            await send(PDToken(req.group_req_id, req.group_req_id, text, meta, status))
    except Exception as e:
        traceback.print_exc()
        from ..core.objs.req import FinishStatus

        await send(PDToken(req.group_req_id, req.group_req_id, "", {"error": str(e)}, FinishStatus.FINISHED_ERROR))


async def pd_master_link(g, master_url: str, connect=None):
    if connect is None:
        import websockets

        connect = lambda url: websockets.connect(url, max_size=ws_max_size(), ping_interval=20)  # noqa: E731
    args = g.args
    reg = PDRegister(node_id_of(args), f"{args.host}:{args.port}", args.run_mode, args.to_dict())
    while True:
        try:
            async with connect(f"{master_url}/pd_register") as ws:
                await ws.send(pickle.dumps(reg))
                lock = asyncio.Lock()

                async def send(obj):
                    async with lock:
                        await ws.send(pickle.dumps(obj))

                async def beat():
                    while True:
                        await send(PDHeartbeat(reg.node_id, _run_status(g)))
                        await asyncio.sleep(HEARTBEAT_S)

                hb = asyncio.create_task(beat())
                try:
                    async for frame in ws:
                        obj = pickle.loads(frame)
                        if isinstance(obj, PDRequest):
                            asyncio.create_task(serve_request(g, obj, send))
                        elif isinstance(obj, tuple) and obj[0] == "ABORT":
                            await g.httpserver_manager.abort_by_master_id(obj[1])
                        elif isinstance(obj, tuple) and obj[0] == "FLUSH_CACHE":
                            await g.httpserver_manager.flush_cache()
                        elif isinstance(obj, tuple) and obj[0] == "RL":
                            await g.httpserver_manager.rl_op(*obj[1])
                        elif isinstance(obj, tuple) and obj[0] == "PROFILER":
                            await g.httpserver_manager.profiler_cmd(obj[1])
                finally:
                    hb.cancel()
        except asyncio.CancelledError:
            raise
        except Exception as e:
            print(f"[pd_loop] link to {master_url} lost ({type(e).__name__}: {e}); retry in {RETRY_S}s", flush=True)
        await asyncio.sleep(RETRY_S)


async def kv_status_link(g, master_url: str, queue: "asyncio.Queue[UpKVStatus]", connect=None):
    """Decode nodes: forward the model ranks' "all pages arrived" notes to the master."""
    if connect is None:
        import websockets

        connect = lambda url: websockets.connect(url, max_size=ws_max_size())  # noqa: E731
    while True:
        try:
            async with connect(f"{master_url}/kv_move_status") as ws:
                while True:
                    up = await queue.get()
                    await ws.send(pickle.dumps(up))
        except asyncio.CancelledError:
            raise
        except Exception:
            await asyncio.sleep(RETRY_S)


async def kv_status_pump(g, queues):
    """Decode nodes: rank 0 of the model pushes (group_req_id, ok) over zmq when a transfer is complete.  `queues`
    maps each master to its upload queue; a note goes to every master (one that does not know the request drops
    it)."""
    import zmq
    import zmq.asyncio

    sock = zmq.asyncio.Context.instance().socket(zmq.PULL)
    sock.bind(f"tcp://127.0.0.1:{g.args.pd_kv_status_port}")
    while True:
        gid, ok = await sock.recv_pyobj()
        for q in list(queues.values()):
            await q.put(UpKVStatus(gid, ok=ok))


def _link_master(g, url: str, queues: dict) -> list:
    tasks = [asyncio.create_task(pd_master_link(g, url))]
    if g.args.run_mode == "decode":
        queues[url] = asyncio.Queue()
        tasks.append(asyncio.create_task(kv_status_link(g, url, queues[url])))
    return tasks


async def follow_config_server(g, queues: dict, links: dict, fetch=None, every_s: float = 10.0):
    """Keeps one link per pd_master that the config server lists (`/registered_objects`); masters that leave the
    list are let go.  Reference: httpserver/pd_loop.py (its loop over the registered pd_masters)."""
    import base64

    args = g.args

    def http_fetch():
        import requests

        r = requests.get(f"http://{args.config_server_host}:{args.config_server_port}/registered_objects", timeout=10)
        r.raise_for_status()
        return pickle.loads(base64.b64decode(r.json()["data"]))

    fetch = fetch or http_fetch
    while True:
        try:
            listed = {f"ws://{m.host_ip_port}" for m in await asyncio.to_thread(fetch)}
        except Exception as e:  # noqa: BLE001
            print(f"[pd_loop] cannot list the pd_masters ({type(e).__name__}: {e})", flush=True)
            listed = None
        if listed is not None:
            for url in listed - set(links):
                links[url] = _link_master(g, url, queues)
            for url in set(links) - listed:
                for t in links.pop(url):
                    t.cancel()
                queues.pop(url, None)
        await asyncio.sleep(every_s)


def start_pd_loops(g):
    args = g.args
    queues, links = {}, {}
    g.kv_status_queues, g.pd_master_links = queues, links
    tasks = []
    if getattr(args, "config_server_host", None) and getattr(args, "config_server_port", None):
        tasks.append(asyncio.create_task(follow_config_server(g, queues, links)))
    else:
        url = f"ws://{args.pd_master_ip}:{args.pd_master_port}"
        links[url] = _link_master(g, url, queues)
        tasks += links[url]
    if args.run_mode == "decode" and args.pd_kv_status_port:
        tasks.append(asyncio.create_task(kv_status_pump(g, queues)))
    return tasks
