"""OpenAI Responses API (/v1/responses) over generate(): `input` (string or message list) plus
`instructions`, non-streaming and the streaming event sequence (response.created,
response.output_text.delta, response.completed).  Reference: lightllm/server/api_responses.py.
"""
from __future__ import annotations

import json
import time
import uuid
from types import SimpleNamespace

from fastapi import Request
from .api_stream_obj import stream_response
from fastapi.responses import JSONResponse, StreamingResponse

from .build_prompt import build_prompt
from .core.objs.sampling_params import SamplingParams


def _messages(body):
    msgs = []
    if body.get("instructions"):
        msgs.append({"role": "system", "content": body["instructions"]})
    inp = body.get("input", "")
    if isinstance(inp, str):
        msgs.append({"role": "user", "content": inp})
    else:
        for item in inp:
            c = item.get("content", "")
            if isinstance(c, list):
                c = "".join(p.get("text", "") for p in c if isinstance(p, dict))
            msgs.append({"role": item.get("role", "user"), "content": c})
    return msgs


async def responses_impl(raw: Request, g):
    body = await raw.json()
    req = SimpleNamespace(messages=_messages(body), character_settings=None, role_settings=None,
                          chat_template_kwargs=None)
    prompt = await build_prompt(req, None)
    mgr = g.httpserver_manager
    t = body.get("temperature", 1.0)
    sp = SamplingParams().init(tokenizer=mgr.tokenizer, max_new_tokens=int(body.get("max_output_tokens") or 4096),
                               do_sample=(t or 0) > 0, temperature=t or 1.0, top_p=body.get("top_p", 1.0),
                               add_special_tokens=False).verify(g.args.vocab_size)
    gen = mgr.generate(prompt, sp, None, raw)
    rid = f"resp_{uuid.uuid4().hex}"
    model = body.get("model", g.args.model_name)

    def envelope(status, text, n_in, n_out):
        return {"id": rid, "object": "response", "created_at": int(time.time()), "status": status, "model": model,
                "output": [{"type": "message", "id": f"msg_{rid[5:29]}", "role": "assistant", "status": status,
                            "content": [{"type": "output_text", "text": text, "annotations": []}]}],
                "usage": {"input_tokens": n_in, "output_tokens": n_out, "total_tokens": n_in + n_out}}

    if not body.get("stream"):
        text, n_in, n_out = [], 0, 0
        async for _, piece, meta, fs in gen:
            text.append(piece)
            n_out += 1
            n_in = meta.get("prompt_tokens", n_in)
        return JSONResponse(envelope("completed", "".join(text), n_in, n_out))

    async def stream():
        text, n_in, n_out = [], 0, 0
        yield f"event: response.created\ndata: {json.dumps({'type': 'response.created', 'response': envelope('in_progress', '', 0, 0)})}\n\n".encode()
        async for _, piece, meta, fs in gen:
            text.append(piece)
            n_out += 1
            n_in = meta.get("prompt_tokens", n_in)
            if piece:
                d = {"type": "response.output_text.delta", "output_index": 0, "content_index": 0, "delta": piece}
                yield f"event: response.output_text.delta\ndata: {json.dumps(d, ensure_ascii=False)}\n\n".encode()
        done = {"type": "response.completed", "response": envelope("completed", "".join(text), n_in, n_out)}
        yield f"event: response.completed\ndata: {json.dumps(done, ensure_ascii=False)}\n\n".encode()

    return await stream_response(stream(), g)
