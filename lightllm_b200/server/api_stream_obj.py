"""Streaming responses whose HTTP status can still say "busy".

An event stream is produced by an async generator that does not run until the response body is iterated, i.e.
after the status line and headers (HTTP 200) are on the wire.  On a pd_master the first iteration is where the
(prefill, decode) pair is chosen and admission may be refused: that has to become HTTP 429, not a 200 with a
broken body.  `stream_response` therefore pulls the first chunk BEFORE it builds the response object when the
server runs as pd_master: a `ServerBusyError` (or a parameter error) raised on the way to the first chunk
propagates to the route's error handling like in a non-streaming route; once a first chunk exists the response
starts normally with that chunk followed by the rest of the same generator.  All other run modes keep the
immediate response start, so that header time-outs of clients and proxies do not count the first token's latency.

Reference: lightllm/server/api_stream_obj.py:30-83 (there a StreamingResponse subclass that withholds the ASGI
`http.response.start` message; here the generator is primed before the response exists).
"""
from __future__ import annotations

from typing import AsyncIterator

from fastapi.responses import StreamingResponse


async def _primed(first, rest: AsyncIterator):
    yield first
    async for chunk in rest:
        yield chunk


async def stream_response(body: AsyncIterator, g=None, media_type: str = "text/event-stream", prime=None,
                          **kw) -> StreamingResponse:
    """`prime`: None = decide from the run mode (pd_master primes), True / False = force."""
    if prime is None:
        prime = getattr(getattr(g, "args", None), "run_mode", "normal") == "pd_master"
    if not prime:
        return StreamingResponse(body, media_type=media_type, **kw)
    it = body.__aiter__()
    try:
        first = await it.__anext__()
    except StopAsyncIteration:          # an empty stream is still a valid (empty) response

        async def _empty():
            return
            yield b""  # pragma: no cover

        return StreamingResponse(_empty(), media_type=media_type, **kw)
    return StreamingResponse(_primed(first, it), media_type=media_type, **kw)
