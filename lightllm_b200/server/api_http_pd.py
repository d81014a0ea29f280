"""Websocket control plane of PD disaggregation.  On the pd_master: `/pd_register` (a node registers, then keeps
the socket open: heartbeats and token uploads flow up, requests flow down) and `/kv_move_status` (decode nodes
report finished KV transfers).  Frames are pickled objects of `pd_io_struct`.
Reference: lightllm/server/api_http_pd.py:26-80.
"""
from __future__ import annotations

import pickle

from fastapi import WebSocket, WebSocketDisconnect

from .pd_io_struct import PDRegister, UpKVStatus


def add_pd_routes(app, g):
    if g.args.run_mode != "pd_master":
        return  # P and D nodes are websocket clients (httpserver/pd_loop.py); they serve no PD routes

    @app.websocket("/pd_register")
    async def pd_register(websocket: WebSocket):
        await websocket.accept()
        mgr = g.httpserver_manager
        node_id = None
        try:
            reg = pickle.loads(await websocket.receive_bytes())
            if not isinstance(reg, PDRegister):
                await websocket.close(code=1003)
                return
            node_id = reg.node_id
            await mgr.register_pd(reg, websocket)
            while True:
                await mgr.on_node_message(pickle.loads(await websocket.receive_bytes()))
        except WebSocketDisconnect:
            pass
        finally:
            if node_id is not None:
                await mgr.remove_pd(node_id)

    @app.websocket("/kv_move_status")
    async def kv_move_status(websocket: WebSocket):
        await websocket.accept()
        mgr = g.httpserver_manager
        try:
            while True:
                up = pickle.loads(await websocket.receive_bytes())
                if isinstance(up, UpKVStatus):
                    await mgr.update_kv_move_status(up)
        except WebSocketDisconnect:
            pass
