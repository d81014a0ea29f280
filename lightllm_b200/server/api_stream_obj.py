"""Streaming responses whose HTTP status can still say "busy".

An event stream is produced by an async generator that does not run until the response body is iterated, i.e.
after the status line and headers (HTTP 200) are on the wire.  On a pd_master the first iteration is where the
(prefill, decode) pair is chosen and admission may be refused: that has to become HTTP 429, not a 200 with a
broken body.  `stream_response` therefore pulls the first chunk BEFORE it builds the response object when the
server runs as pd_master: a `ServerBusyError` (or a parameter error) raised on the way to the first chunk
propagates to the route's error handling like in a non-streaming route; once a first chunk exists the response
starts normally with that chunk followed by the rest of the same generator.  In the other run modes admission
is refused within about two seconds (no free request slot) while the first token of a long prompt may take much
longer, so there the first chunk is awaited for a short while only (`EARLY_S`): an error raised in that window
still becomes a proper status code, otherwise the response starts and the pending first chunk follows, so that
header time-outs of clients and proxies do not count the first token's latency.

Reference: lightllm/server/api_stream_obj.py:30-83 (there a StreamingResponse subclass that withholds the ASGI
`http.response.start` message; here the generator is primed before the response exists).
"""
from __future__ import annotations

from typing import AsyncIterator

from fastapi.responses import StreamingResponse


EARLY_S = 2.5     # longer than the wait for a free request slot (2 s)


async def _after(task, rest: AsyncIterator):
    try:
        yield await task
    except StopAsyncIteration:
        return
    async for chunk in rest:
        yield chunk


async def _primed(first, rest: AsyncIterator):
    yield first
    async for chunk in rest:
        yield chunk


async def stream_response(body: AsyncIterator, g=None, media_type: str = "text/event-stream", prime=None,
                          **kw) -> StreamingResponse:
    """`prime`: None = decide from the run mode (pd_master waits for the first chunk, the other modes for at most
    EARLY_S), True = always wait for the first chunk, False = start at once."""
    if prime is None:
        prime = True if getattr(getattr(g, "args", None), "run_mode", "normal") == "pd_master" else None
    if prime is False:
        return StreamingResponse(body, media_type=media_type, **kw)
    it = body.__aiter__()
    if not prime:                       # other run modes: wait a short while for an early refusal
        import asyncio

        async def first_chunk():       # (asyncio.ensure_future wants a coroutine, __anext__ gives an awaitable)
            return await it.__anext__()

        task = asyncio.ensure_future(first_chunk())
        done, _ = await asyncio.wait({task}, timeout=EARLY_S)
        if done:
            exc = task.exception()
            if exc is not None and not isinstance(exc, StopAsyncIteration):
                raise exc
        return StreamingResponse(_after(task, it), media_type=media_type, **kw)
    try:
        first = await it.__anext__()
    except StopAsyncIteration:          # an empty stream is still a valid (empty) response

        async def _empty():
            return
            yield b""  # pragma: no cover

        return StreamingResponse(_empty(), media_type=media_type, **kw)
    return StreamingResponse(_primed(first, it), media_type=media_type, **kw)
