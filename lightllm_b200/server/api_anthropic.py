"""Anthropic Messages API (/v1/messages, /v1/messages/count_tokens) over the same generate() generator.
Maps system + messages (text and tool_result blocks) to the chat template, streams the Anthropic event
sequence (message_start, content_block_start/delta/stop, message_delta, message_stop).
Reference: lightllm/server/api_anthropic.py.
"""
from __future__ import annotations

import json
import uuid
from types import SimpleNamespace

from fastapi import Request
from .api_stream_obj import stream_response
from fastapi.responses import JSONResponse, StreamingResponse

from .build_prompt import build_prompt
from .core.objs.sampling_params import SamplingParams

_STOP = {"stop": "end_turn", "length": "max_tokens", "abort": "end_turn", "error": "end_turn"}


def _text_of(content) -> str:
    if isinstance(content, str):
        return content
    out = []
    for blk in content or []:
        t = blk.get("type")
        if t == "text":
            out.append(blk.get("text", ""))
        elif t == "tool_result":
            out.append(_text_of(blk.get("content", "")))
        elif t == "tool_use":
            out.append(json.dumps({"name": blk.get("name"), "arguments": blk.get("input", {})}))
    return "".join(out)


def _to_chat(body: dict):
    msgs = []
    if body.get("system"):
        msgs.append({"role": "system", "content": _text_of(body["system"])})
    for m in body.get("messages", []):
        msgs.append({"role": m.get("role", "user"), "content": _text_of(m.get("content"))})
    tools = None
    if body.get("tools"):
        tools = [{"name": t["name"], "description": t.get("description"), "parameters": t.get("input_schema")}
                 for t in body["tools"]]
    return msgs, tools


async def _prompt(body):
    msgs, tools = _to_chat(body)
    req = SimpleNamespace(messages=msgs, character_settings=None, role_settings=None, chat_template_kwargs=None)
    return await build_prompt(req, tools)


def _sampling(body, tokenizer, vocab):
    sp = SamplingParams().init(tokenizer=tokenizer, max_new_tokens=int(body.get("max_tokens", 1024)),
                               do_sample=body.get("temperature", 1.0) > 0, temperature=body.get("temperature", 1.0),
                               top_p=body.get("top_p", 1.0), top_k=body.get("top_k", -1) or -1,
                               stop_sequences=body.get("stop_sequences"), add_special_tokens=False)
    return sp.verify(vocab)


async def anthropic_count_tokens_impl(raw: Request, g):
    body = await raw.json()
    prompt = await _prompt(body)
    return JSONResponse({"input_tokens": g.httpserver_manager.tokens(prompt)})


async def anthropic_messages_impl(raw: Request, g):
    body = await raw.json()
    prompt = await _prompt(body)
    mgr = g.httpserver_manager
    sp = _sampling(body, mgr.tokenizer, g.args.vocab_size)
    gen = mgr.generate(prompt, sp, None, raw)
    msg_id = f"msg_{uuid.uuid4().hex[:24]}"
    model = body.get("model", g.args.model_name)
    if not body.get("stream"):
        text, n_out, n_in, reason = [], 0, 0, None
        async for _, piece, meta, fs in gen:
            text.append(piece)
            n_out += 1
            n_in = meta.get("prompt_tokens", n_in)
            if fs.is_finished():
                reason = fs.get_finish_reason()
        return JSONResponse({"id": msg_id, "type": "message", "role": "assistant", "model": model,
                             "content": [{"type": "text", "text": "".join(text)}],
                             "stop_reason": _STOP.get(reason, "end_turn"), "stop_sequence": None,
                             "usage": {"input_tokens": n_in, "output_tokens": n_out}})

    def ev(name, data):
        return f"event: {name}\ndata: {json.dumps(data, ensure_ascii=False)}\n\n".encode()

    async def stream():
        started, n_out, n_in, reason = False, 0, 0, None
        async for _, piece, meta, fs in gen:
            n_in = meta.get("prompt_tokens", n_in)
            if not started:
                started = True
                yield ev("message_start", {"type": "message_start", "message": {
                    "id": msg_id, "type": "message", "role": "assistant", "model": model, "content": [],
                    "stop_reason": None, "usage": {"input_tokens": n_in, "output_tokens": 0}}})
                yield ev("content_block_start", {"type": "content_block_start", "index": 0,
                                                 "content_block": {"type": "text", "text": ""}})
            n_out += 1
            if piece:
                yield ev("content_block_delta", {"type": "content_block_delta", "index": 0,
                                                 "delta": {"type": "text_delta", "text": piece}})
            if fs.is_finished():
                reason = fs.get_finish_reason()
        yield ev("content_block_stop", {"type": "content_block_stop", "index": 0})
        yield ev("message_delta", {"type": "message_delta", "delta": {"stop_reason": _STOP.get(reason, "end_turn"),
                                                                       "stop_sequence": None},
                                   "usage": {"output_tokens": n_out}})
        yield ev("message_stop", {"type": "message_stop"})

    return await stream_response(stream(), g)
