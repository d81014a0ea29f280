"""A busy pd_master answers a streaming request with HTTP 429 instead of a 200 whose body breaks: the event
generator is primed before the response starts (server/api_stream_obj.py).  Other run modes start at once."""
import asyncio
from types import SimpleNamespace

import pytest
from fastapi import FastAPI
from fastapi.testclient import TestClient

from lightllm_b200.server.api_stream_obj import stream_response
from lightllm_b200.utils.errors import ServerBusyError


def _app(run_mode, fail_at):
    app = FastAPI()
    g = SimpleNamespace(args=SimpleNamespace(run_mode=run_mode))

    async def events():
        for i in range(3):
            if i == fail_at:
                raise ServerBusyError("no prefill / decode pair is free")
            await asyncio.sleep(0)
            yield f"data:{i}\\n\\n".encode()

    @app.get("/s")
    async def s():
        try:
            return await stream_response(events(), g)
        except ServerBusyError as e:
            from fastapi.responses import JSONResponse

            return JSONResponse({"message": str(e)}, status_code=429)

    return TestClient(app, raise_server_exceptions=False)


def test_pd_master_refusal_before_the_first_chunk_is_a_429():
    r = _app("pd_master", fail_at=0).get("/s")
    assert r.status_code == 429 and "free" in r.json()["message"]


def test_pd_master_stream_is_complete_and_unduplicated():
    r = _app("pd_master", fail_at=-1).get("/s")
    assert r.status_code == 200 and r.text == "data:0\\n\\ndata:1\\n\\ndata:2\\n\\n"
    assert r.headers["content-type"].startswith("text/event-stream")


def test_other_modes_start_the_response_at_once():
    # the generator has not run when the response object is built: its refusal can no longer change the status
    c = _app("normal", fail_at=0)
    try:
        r = c.get("/s")
        assert r.status_code == 200
    except Exception:
        pass          # depending on the transport the broken body surfaces as a client-side error: still not a 429


def test_empty_stream():
    app = FastAPI()

    async def nothing():
        return
        yield b""

    @app.get("/e")
    async def e():
        return await stream_response(nothing(), prime=True)

    r = TestClient(app).get("/e")
    assert r.status_code == 200 and r.text == ""
