"""Anthropic Messages API (/v1/messages, /v1/messages/count_tokens) as a translation layer over the chat-completions
route: the request becomes a chat request (system blocks, text / tool_use / tool_result / thinking blocks, tools and
tool_choice), the answer comes back as content blocks (thinking, text, tool_use) with Anthropic stop reasons, and a
streamed answer is re-cut into the Anthropic event sequence (message_start, content_block_start / delta / stop per
block with text_delta, thinking_delta or input_json_delta, message_delta, message_stop).  Tool calls and reasoning
therefore go through the same parsers (`--tool_call_parser`, `--reasoning_parser`) as the OpenAI route.

Reference: lightllm/server/api_anthropic.py (same approach: Anthropic -> chat request -> chat response ->
Anthropic; PDF documents are not converted here).
"""
from __future__ import annotations

import json
import uuid
from types import SimpleNamespace
from typing import Any, AsyncIterator, Dict, List, Optional

from fastapi import Request
from fastapi.responses import JSONResponse

from .api_stream_obj import stream_response
from .build_prompt import build_prompt

STOP_REASON = {"stop": "end_turn", "length": "max_tokens", "tool_calls": "tool_use", "abort": "end_turn",
               "error": "end_turn", None: "end_turn"}


def anthropic_error(status: int, message: str, kind: str = "invalid_request_error") -> JSONResponse:
    return JSONResponse({"type": "error", "error": {"type": kind, "message": message}}, status_code=status)


# ---------------------------------------------------------------------------- request -> chat request
def _text_of(content) -> str:
    if isinstance(content, str):
        return content
    out = []
    for blk in content or []:
        if isinstance(blk, str):
            out.append(blk)
        elif blk.get("type") == "text":
            out.append(blk.get("text", ""))
        elif blk.get("type") == "tool_result":
            out.append(_text_of(blk.get("content", "")))
    return "".join(out)


def to_chat_request(body: Dict[str, Any]) -> Dict[str, Any]:
    """The chat-completions request (a plain dict) that asks for the same thing as the Messages request `body`."""
    msgs: List[Dict[str, Any]] = []
    if body.get("system"):
        msgs.append({"role": "system", "content": _text_of(body["system"])})
    for m in body.get("messages", []):
        role, content = m.get("role", "user"), m.get("content")
        if isinstance(content, str):
            msgs.append({"role": role, "content": content})
            continue
        text, calls, thinking, pending = [], [], [], []
        for blk in content or []:
            t = blk.get("type")
            if t == "text":
                text.append(blk.get("text", ""))
            elif t == "thinking":
                thinking.append(blk.get("thinking", ""))
            elif t == "tool_use":
                calls.append({"id": blk.get("id") or f"toolu_{uuid.uuid4().hex[:24]}", "type": "function",
                              "function": {"name": blk.get("name"),
                                           "arguments": json.dumps(blk.get("input") or {}, ensure_ascii=False)}})
            elif t == "tool_result":
                # a tool result is its own message in the chat format; text before it stays with the user turn
                if text:
                    msgs.append({"role": role, "content": "".join(text)})
                    text = []
                pending.append({"role": "tool", "tool_call_id": blk.get("tool_use_id"),
                                "content": _text_of(blk.get("content", ""))})
            elif t == "image":
                src = blk.get("source") or {}
                url = src.get("url") if src.get("type") == "url" else \
                    f"data:{src.get('media_type', 'image/png')};base64,{src.get('data', '')}"
                text.append("")   # pictures travel as separate parts
                pending.append({"role": role, "content": [{"type": "image_url", "image_url": {"url": url}}]})
        msgs.extend(p for p in pending if p["role"] == "tool")
        if text or calls or thinking:
            msg: Dict[str, Any] = {"role": role, "content": "".join(text)}
            if calls:
                msg["tool_calls"] = calls
            if thinking:
                msg["reasoning_content"] = "".join(thinking)
            msgs.append(msg)
        msgs.extend(p for p in pending if p["role"] != "tool")
    out: Dict[str, Any] = {"model": body.get("model", "default_model_name"), "messages": msgs,
                           "max_tokens": int(body.get("max_tokens", 1024)), "stream": bool(body.get("stream"))}
    t = body.get("temperature")
    if t is not None:
        out["temperature"] = t if t > 0 else 1.0
        out["do_sample"] = t > 0
    for src, dst in (("top_p", "top_p"), ("top_k", "top_k"), ("stop_sequences", "stop")):
        if body.get(src) is not None:
            out[dst] = body[src]
    if body.get("tools"):
        out["tools"] = [{"type": "function", "function": {"name": t["name"], "description": t.get("description"),
                                                            "parameters": t.get("input_schema") or {}}}
                        for t in body["tools"] if t.get("name")]
        choice = body.get("tool_choice") or {"type": "auto"}
        kind = choice.get("type", "auto")
        if kind == "any":
            out["tool_choice"] = "required"
        elif kind == "tool":
            out["tool_choice"] = {"type": "function", "function": {"name": choice.get("name")}}
        elif kind == "none":
            out["tool_choice"] = "none"
        else:
            out["tool_choice"] = "auto"
        if choice.get("disable_parallel_tool_use"):
            out["parallel_tool_calls"] = False
    thinking = body.get("thinking")
    if isinstance(thinking, dict):
        on = thinking.get("type") == "enabled"
        out["chat_template_kwargs"] = {"enable_thinking": on, "thinking": on}
        out["separate_reasoning"] = True
    if out["stream"]:
        out["stream_options"] = {"include_usage": True}
    return out


# ---------------------------------------------------------------------------- chat response -> message
def _tool_input(arguments) -> Any:
    if isinstance(arguments, (dict, list)):
        return arguments
    try:
        return json.loads(arguments) if arguments else {}
    except (TypeError, ValueError):
        return {"_raw": arguments}


def chat_response_to_message(resp: Dict[str, Any], model: str, msg_id: Optional[str] = None) -> Dict[str, Any]:
    choice = (resp.get("choices") or [{}])[0]
    msg = choice.get("message") or {}
    content: List[Dict[str, Any]] = []
    if msg.get("reasoning_content"):
        content.append({"type": "thinking", "thinking": msg["reasoning_content"], "signature": ""})
    if msg.get("content"):
        content.append({"type": "text", "text": msg["content"]})
    for c in msg.get("tool_calls") or []:
        f = c.get("function") or {}
        content.append({"type": "tool_use", "id": (c.get("id") or f"call_{uuid.uuid4().hex[:24]}").replace("call_", "toolu_", 1),
                        "name": f.get("name"), "input": _tool_input(f.get("arguments"))})
    if not content:
        content.append({"type": "text", "text": ""})
    usage = resp.get("usage") or {}
    cached = ((usage.get("prompt_tokens_details") or {}).get("cached_tokens")) or 0
    return {"id": msg_id or f"msg_{uuid.uuid4().hex[:24]}", "type": "message", "role": "assistant", "model": model,
            "content": content, "stop_reason": STOP_REASON.get(choice.get("finish_reason"), "end_turn"),
            "stop_sequence": None,
            "usage": {"input_tokens": usage.get("prompt_tokens", 0), "output_tokens": usage.get("completion_tokens", 0),
                      "cache_read_input_tokens": cached, "cache_creation_input_tokens": 0}}


# ---------------------------------------------------------------------------- chat stream -> event stream
def _ev(name: str, data: Dict[str, Any]) -> bytes:
    return f"event: {name}\ndata: {json.dumps(data, ensure_ascii=False)}\n\n".encode()


async def chat_chunks_to_events(chunks: AsyncIterator[Dict[str, Any]], model: str,
                                msg_id: Optional[str] = None) -> AsyncIterator[bytes]:
    """Re-cuts chat-completion stream chunks (dicts) into Anthropic events.  One content block is open at a time:
    reasoning opens a thinking block, text a text block, every tool call (by its index) a tool_use block whose
    arguments arrive as input_json_delta pieces."""
    msg_id = msg_id or f"msg_{uuid.uuid4().hex[:24]}"
    started = False
    index = -1                 # index of the open block
    open_kind: Optional[str] = None      # "thinking" | "text" | ("tool", tool index)
    finish, usage = None, {}

    def start_message(prompt_tokens=0):
        return _ev("message_start", {"type": "message_start", "message": {
            "id": msg_id, "type": "message", "role": "assistant", "model": model, "content": [], "stop_reason": None,
            "stop_sequence": None, "usage": {"input_tokens": prompt_tokens, "output_tokens": 0}}})

    def close():
        nonlocal open_kind
        out = []
        if open_kind is not None:
            out.append(_ev("content_block_stop", {"type": "content_block_stop", "index": index}))
            open_kind = None
        return out

    def open_block(kind, block):
        nonlocal index, open_kind
        out = close()
        index += 1
        open_kind = kind
        out.append(_ev("content_block_start", {"type": "content_block_start", "index": index, "content_block": block}))
        return out

    async for chunk in chunks:
        if not started:
            started = True
            yield start_message()
        if chunk.get("usage"):
            usage = chunk["usage"]
        for choice in chunk.get("choices") or []:
            delta = choice.get("delta") or {}
            if delta.get("reasoning_content"):
                if open_kind != "thinking":
                    for e in open_block("thinking", {"type": "thinking", "thinking": ""}):
                        yield e
                yield _ev("content_block_delta", {"type": "content_block_delta", "index": index,
                                                  "delta": {"type": "thinking_delta",
                                                            "thinking": delta["reasoning_content"]}})
            if delta.get("content"):
                if open_kind != "text":
                    for e in open_block("text", {"type": "text", "text": ""}):
                        yield e
                yield _ev("content_block_delta", {"type": "content_block_delta", "index": index,
                                                  "delta": {"type": "text_delta", "text": delta["content"]}})
            for c in delta.get("tool_calls") or []:
                f = c.get("function") or {}
                kind = ("tool", c.get("index", 0))
                if f.get("name") or open_kind != kind:      # a call announces itself with its name
                    tid = (c.get("id") or f"call_{uuid.uuid4().hex[:24]}").replace("call_", "toolu_", 1)
                    for e in open_block(kind, {"type": "tool_use", "id": tid, "name": f.get("name") or "",
                                               "input": {}}):
                        yield e
                if f.get("arguments"):
                    yield _ev("content_block_delta", {"type": "content_block_delta", "index": index,
                                                      "delta": {"type": "input_json_delta",
                                                                "partial_json": f["arguments"]}})
            if choice.get("finish_reason"):
                finish = choice["finish_reason"]
    if not started:
        yield start_message()
    if index < 0:              # an empty answer still has one (empty) text block
        index, open_kind = 0, "text"
        yield _ev("content_block_start", {"type": "content_block_start", "index": 0,
                                          "content_block": {"type": "text", "text": ""}})
    for e in close():
        yield e
    yield _ev("message_delta", {"type": "message_delta",
                                "delta": {"stop_reason": STOP_REASON.get(finish, "end_turn"), "stop_sequence": None},
                                "usage": {"input_tokens": usage.get("prompt_tokens", 0),
                                          "output_tokens": usage.get("completion_tokens", 0)}})
    yield _ev("message_stop", {"type": "message_stop"})


async def sse_to_chunks(body_iterator) -> AsyncIterator[Dict[str, Any]]:
    """`data: {...}` lines of a chat-completion stream as dicts (ends at `data: [DONE]`)."""
    buf = b""
    async for part in body_iterator:
        buf += part if isinstance(part, bytes) else part.encode()
        while b"\n\n" in buf:
            line, buf = buf.split(b"\n\n", 1)
            line = line.strip()
            if not line.startswith(b"data:"):
                continue
            payload = line[5:].strip()
            if payload == b"[DONE]":
                return
            yield json.loads(payload)


# ---------------------------------------------------------------------------- routes
async def anthropic_count_tokens_impl(raw: Request, g):
    body = await raw.json()
    chat = to_chat_request(body)
    tools = [t["function"] for t in chat.get("tools", [])] or None
    req = SimpleNamespace(messages=chat["messages"], character_settings=None, role_settings=None,
                          chat_template_kwargs=chat.get("chat_template_kwargs"))
    prompt = await build_prompt(req, tools)
    return JSONResponse({"input_tokens": g.httpserver_manager.tokens(prompt)})


async def anthropic_messages_impl(raw: Request, g):
    from .api_models import ChatCompletionRequest
    from .api_openai import chat_completions_impl

    try:
        body = await raw.json()
    except ValueError:
        return anthropic_error(400, "the request body is not JSON")
    if not isinstance(body.get("messages"), list) or not body["messages"]:
        return anthropic_error(400, "messages: a non-empty list is required")
    model = body.get("model", g.args.model_name)
    try:
        request = ChatCompletionRequest(**to_chat_request(body))
    except Exception as e:
        return anthropic_error(400, f"invalid request: {e}")
    resp = await chat_completions_impl(request, raw, g)
    msg_id = f"msg_{uuid.uuid4().hex[:24]}"
    if getattr(resp, "body_iterator", None) is not None:          # streamed
        if resp.status_code != 200:
            return resp
        return await stream_response(chat_chunks_to_events(sse_to_chunks(resp.body_iterator), model, msg_id), g)
    payload = json.loads(bytes(resp.body))
    if resp.status_code != 200:
        err = payload.get("error") or payload
        return anthropic_error(resp.status_code, str(err.get("message", err)),
                               "overloaded_error" if resp.status_code in (429, 503) else "invalid_request_error")
    return JSONResponse(chat_response_to_message(payload, model, msg_id))
