"""RL control plane (enabled by --enable_rl): a trainer pauses admission, flushes the prefix cache,
releases / resumes GPU memory and pushes new weights without restarting the server.
Routes follow the reference (lightllm/server/api_http_rl.py:51-143).
"""
from __future__ import annotations

from fastapi import Request
from fastapi.responses import JSONResponse


def add_rl_routes(app, g):
    mgr = lambda: g.httpserver_manager  # noqa: E731

    @app.post("/abort_request")
    async def abort_request(request: Request):
        body = await request.json()
        if body.get("abort_all"):
            await mgr().abort_all()
            return {"success": True}
        ok = await mgr().abort(int(body["request_id"]))
        return {"success": bool(ok)}

    @app.post("/pause_generation")
    async def pause_generation():
        mgr().paused = True
        await mgr().abort_all()
        return {"success": True}

    @app.post("/continue_generation")
    async def continue_generation():
        mgr().paused = False
        return {"success": True}

    @app.post("/flush_cache")
    async def flush_cache():
        await mgr().flush_cache()
        return {"success": True}

    @app.post("/release_memory_occupation")
    async def release_memory(request: Request):
        body = await request.json() if (await request.body()) else {}
        await mgr().rl_op("release_memory_occupation", {"tags": body.get("tags") or ["kv_cache"]})
        return {"success": True}

    @app.post("/resume_memory_occupation")
    async def resume_memory(request: Request):
        body = await request.json() if (await request.body()) else {}
        await mgr().rl_op("resume_memory_occupation", {"tags": body.get("tags") or ["kv_cache"]})
        return {"success": True}

    @app.post("/init_weights_update_group")
    async def init_group(request: Request):
        await mgr().rl_op("init_weights_update_group", await request.json())
        return {"success": True}

    @app.post("/destroy_weights_update_group")
    async def destroy_group(request: Request):
        await mgr().rl_op("destroy_weights_update_group", await request.json())
        return {"success": True}

    @app.post("/update_weights_from_disk")
    async def update_from_disk(request: Request):
        body = await request.json()
        await mgr().rl_op("update_weights_from_disk", body)
        if body.get("weight_version"):
            g.args.weight_version = body["weight_version"]
        return {"success": True}

    @app.post("/update_weights_from_tensor")
    async def update_from_tensor(request: Request):
        import base64
        import io

        import torch

        body = await request.json()
        named = [(n, torch.load(io.BytesIO(base64.b64decode(b)), weights_only=True)) for n, b in body["named_tensors"]]
        await mgr().rl_op("update_weights_from_tensor", {"named_tensors": named, "weight_version": body.get("weight_version")})
        if body.get("weight_version"):
            g.args.weight_version = body["weight_version"]
        return {"success": True}

    @app.post("/update_weights_from_distributed")
    async def update_from_distributed(request: Request):
        await mgr().rl_op("update_weights_from_distributed", await request.json())
        return {"success": True}

    @app.post("/update_weights_from_ipc")
    async def update_from_ipc(request: Request):
        await mgr().rl_op("update_weights_from_ipc", await request.json())
        return {"success": True}
