"""config_server run mode: a small registry for deployments with several pd_masters or remote ViT
nodes.  pd_masters and visual servers register over websockets (the entry lives as long as the socket),
P/D nodes list them over HTTP, every front-end draws disjoint request-id and multimodal-id ranges, and
model ranks can ask it to host a rendezvous TCPStore for their NCCL world.
Reference: lightllm/server/config_server/api_http.py:35-200, nccl_tcp_store.py.
"""
from __future__ import annotations

import asyncio
import base64
import multiprocessing as mp
import pickle
import threading
from typing import Dict, List

from fastapi import FastAPI, Query, WebSocket, WebSocketDisconnect
from fastapi.responses import JSONResponse

app = FastAPI()

REQ_ID_RANGE = 800_000
MM_ID_RANGE = 8_000_000
MM_ID_BASE = 100_000_000


class Registry:
    def __init__(self):
        self.lock = threading.Lock()
        self.pd_masters: Dict[str, object] = {}
        self.visual: Dict[str, object] = {}
        self.next_req_id = 0
        self.next_mm_id = MM_ID_BASE
        self.stores: Dict[int, mp.Process] = {}
        self.store_clients: Dict[int, List[bool]] = {}
        self.store_lock = asyncio.Lock()
        self.host = "0.0.0.0"

    def take_req_ids(self):
        with self.lock:
            if self.next_req_id + REQ_ID_RANGE > 2 ** 63 - 1:
                self.next_req_id = 0
            s = self.next_req_id
            self.next_req_id += REQ_ID_RANGE
            return s, self.next_req_id

    def take_mm_ids(self):
        with self.lock:
            if self.next_mm_id + MM_ID_RANGE > 2 ** 63 - 1:
                self.next_mm_id = MM_ID_BASE
            s = self.next_mm_id
            self.next_mm_id += MM_ID_RANGE
            return s, self.next_mm_id


registry = Registry()


@app.get("/liveness")
@app.post("/liveness")
def liveness():
    return {"status": "ok"}


@app.get("/readiness")
@app.post("/readiness")
def readiness():
    return {"status": "ok"}


@app.get("/healthz")
@app.get("/health")
@app.head("/health")
async def health():
    return JSONResponse({"message": "Ok"}, status_code=200)


async def _hold(websocket: WebSocket, table: Dict[str, object]):
    await websocket.accept()
    obj = pickle.loads(await websocket.receive_bytes())
    key = f"{getattr(obj, 'host_ip_port', None) or getattr(obj, 'node_id', id(obj))}"
    with registry.lock:
        table[key] = obj
    try:
        while True:
            await websocket.receive_text()  # heartbeats
    except (WebSocketDisconnect, RuntimeError):
        pass
    finally:
        with registry.lock:
            table.pop(key, None)


@app.websocket("/pd_master_register")
async def pd_master_register(websocket: WebSocket):
    await _hold(websocket, registry.pd_masters)


@app.websocket("/visual_register")
async def visual_register(websocket: WebSocket):
    await _hold(websocket, registry.visual)


def _dump(table):
    with registry.lock:
        return {"data": base64.b64encode(pickle.dumps(list(table.values()))).decode()}


@app.get("/registered_objects")
async def registered_objects():
    return _dump(registry.pd_masters)


@app.get("/registered_visual_objects")
async def registered_visual_objects():
    return _dump(registry.visual)


@app.get("/allocate_global_unique_id_range")
async def allocate_ids():
    s, e = registry.take_req_ids()
    return {"start_id": s, "end_id": e}


@app.get("/allocate_global_unique_multimodal_id_range")
async def allocate_mm_ids():
    s, e = registry.take_mm_ids()
    return {"start_id": s, "end_id": e}


def _store_main(host: str, port: int):
    import time

    import torch.distributed as dist

    from ...utils.process_utils import start_parent_check_thread

    start_parent_check_thread()
    store = dist.TCPStore(host_name=host, port=port, world_size=None, is_master=True, wait_for_workers=False,
                          multi_tenant=True)
    while True:
        store.num_keys()
        time.sleep(20)


@app.get("/start_tcp_store_server")
async def start_tcp_store_server(tcp_store_port: int = Query(...), rank_id: int = Query(...),
                                 world_size: int = Query(...)):
    """Rank 0 of a model world (re)starts the store on `tcp_store_port`; the other ranks poll until it is up.
    Each rank may claim its slot once per store start, so a restarted world gets a fresh store."""
    async with registry.store_lock:
        if rank_id == 0:
            old = registry.stores.pop(tcp_store_port, None)
            if old is not None:
                old.kill()
                old.join()
            p = mp.get_context("spawn").Process(target=_store_main, args=(registry.host, tcp_store_port), daemon=True)
            p.start()
            registry.stores[tcp_store_port] = p
            st = [True] * world_size
            st[0] = False
            registry.store_clients[tcp_store_port] = st
            return {"status": "ok"}
        st = registry.store_clients.get(tcp_store_port)
        if st is None or rank_id >= len(st) or not st[rank_id]:
            return JSONResponse({"status": "not ready"}, status_code=503)
        st[rank_id] = False
        if not any(st):
            registry.store_clients.pop(tcp_store_port, None)
        return {"status": "ok"}
