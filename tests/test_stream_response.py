"""A busy pd_master answers a streaming request with HTTP 429 instead of a 200 whose body breaks: the event
generator is primed before the response starts (server/api_stream_obj.py).  Other run modes wait for the first chunk
for a short while only (an early refusal still becomes a status code, a slow first token does not hold the headers)."""
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


def test_other_modes_turn_an_early_refusal_into_a_status_code_too():
    # admission is refused within about two seconds (no free request slot): the first chunk is awaited that long
    r = _app("normal", fail_at=0).get("/s")
    assert r.status_code == 429
    r = _app("normal", fail_at=-1).get("/s")
    assert r.status_code == 200 and r.text == "data:0\\n\\ndata:1\\n\\ndata:2\\n\\n"


def test_other_modes_do_not_wait_long_for_a_slow_first_chunk(monkeypatch):
    import time

    from lightllm_b200.server import api_stream_obj as so

    monkeypatch.setattr(so, "EARLY_S", 0.1)
    built = {}

    async def slow():
        await asyncio.sleep(0.6)             # a long prompt: the first token takes longer than the waiting window
        yield b"a"
        yield b"b"

    async def run():
        t0 = time.time()
        resp = await so.stream_response(slow(), SimpleNamespace(args=SimpleNamespace(run_mode="normal")))
        built["after"] = time.time() - t0
        return b"".join([c async for c in resp.body_iterator])

    assert asyncio.run(run()) == b"ab" and built["after"] < 0.4       # the response object existed before the chunk
    # the empty stream and the forced immediate start
    async def nothing():
        return
        yield b""

    async def run2():
        resp = await so.stream_response(nothing(), SimpleNamespace(args=SimpleNamespace(run_mode="normal")))
        return b"".join([c async for c in resp.body_iterator])

    assert asyncio.run(run2()) == b""


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
