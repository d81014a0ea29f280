"""OpenAI Responses API (/v1/responses) as a translation layer over the chat-completions route.

Request: `instructions` + `input` (a string, or items: messages with input_text / output_text / input_image parts,
function_call, function_call_output, reasoning), flat function `tools`, `tool_choice`, `text.format` (json_schema /
json_object), `reasoning`, `max_output_tokens`.  Answer: `output` items in order reasoning, message (output_text),
function_call; `status` completed / incomplete (max_output_tokens).  Stream: response.created,
response.in_progress, then per output item response.output_item.added, the item's deltas
(response.reasoning_summary_text.delta, response.output_text.delta, response.function_call_arguments.delta) and
their .done events, response.output_item.done, and response.completed with the whole response.

Reference: lightllm/server/api_responses.py (same approach: Responses -> chat request -> chat answer -> Responses).
"""
from __future__ import annotations

import json
import time
import uuid
from typing import Any, AsyncIterator, Dict, List, Optional

from fastapi import Request
from fastapi.responses import JSONResponse

from .api_anthropic import sse_to_chunks
from .api_stream_obj import stream_response


# ---------------------------------------------------------------------------- request -> chat request
def _parts_to_chat(parts) -> Any:
    """Content parts of an input message -> a string when they are all text, else chat content parts."""
    if isinstance(parts, str):
        return parts
    out, only_text = [], True
    for p in parts or []:
        if isinstance(p, str):
            out.append({"type": "text", "text": p})
        elif p.get("type") in ("input_text", "output_text", "text"):
            out.append({"type": "text", "text": p.get("text", "")})
        elif p.get("type") == "input_image":
            only_text = False
            out.append({"type": "image_url", "image_url": {"url": p.get("image_url") or p.get("file_id") or ""}})
        elif p.get("type") == "refusal":
            out.append({"type": "text", "text": p.get("refusal", "")})
    return "".join(x["text"] for x in out) if only_text else out


def input_to_messages(body: Dict[str, Any]) -> List[Dict[str, Any]]:
    msgs: List[Dict[str, Any]] = []
    if body.get("instructions"):
        msgs.append({"role": "system", "content": body["instructions"]})
    inp = body.get("input", "")
    if isinstance(inp, str):
        msgs.append({"role": "user", "content": inp})
        return msgs
    pending_reasoning: List[str] = []
    for item in inp or []:
        kind = item.get("type") or ("message" if "role" in item else None)
        if kind == "message":
            role = {"developer": "system"}.get(item.get("role", "user"), item.get("role", "user"))
            m = {"role": role, "content": _parts_to_chat(item.get("content", ""))}
            if role == "assistant" and pending_reasoning:
                m["reasoning_content"], pending_reasoning = "".join(pending_reasoning), []
            msgs.append(m)
        elif kind == "function_call":
            call = {"id": item.get("call_id") or item.get("id") or f"call_{uuid.uuid4().hex[:24]}", "type": "function",
                    "function": {"name": item.get("name"), "arguments": item.get("arguments") or "{}"}}
            if msgs and msgs[-1]["role"] == "assistant":
                msgs[-1].setdefault("tool_calls", []).append(call)
            else:
                m = {"role": "assistant", "content": "", "tool_calls": [call]}
                if pending_reasoning:
                    m["reasoning_content"], pending_reasoning = "".join(pending_reasoning), []
                msgs.append(m)
        elif kind == "function_call_output":
            out = item.get("output")
            msgs.append({"role": "tool", "tool_call_id": item.get("call_id"),
                         "content": out if isinstance(out, str) else json.dumps(out, ensure_ascii=False)})
        elif kind == "reasoning":
            for part in (item.get("summary") or []) + (item.get("content") or []):
                if isinstance(part, dict) and part.get("text"):
                    pending_reasoning.append(part["text"])
    return msgs


def to_chat_request(body: Dict[str, Any]) -> Dict[str, Any]:
    out: Dict[str, Any] = {"model": body.get("model", "default_model_name"), "messages": input_to_messages(body),
                           "stream": bool(body.get("stream"))}
    if body.get("max_output_tokens"):
        out["max_tokens"] = int(body["max_output_tokens"])
    t = body.get("temperature")
    if t is not None:
        out["temperature"] = t if t > 0 else 1.0
        out["do_sample"] = t > 0
    if body.get("top_p") is not None:
        out["top_p"] = body["top_p"]
    tools = [t for t in body.get("tools") or [] if t.get("type", "function") == "function" and t.get("name")]
    if tools:
        out["tools"] = [{"type": "function", "function": {"name": t["name"], "description": t.get("description"),
                                                            "parameters": t.get("parameters") or {}}} for t in tools]
        choice = body.get("tool_choice", "auto")
        if isinstance(choice, dict):
            out["tool_choice"] = {"type": "function", "function": {"name": choice.get("name")}} \
                if choice.get("type") == "function" else "auto"
        elif choice in ("auto", "required", "none"):
            out["tool_choice"] = choice
        if body.get("parallel_tool_calls") is False:
            out["parallel_tool_calls"] = False
    fmt = (body.get("text") or {}).get("format") or {}
    if fmt.get("type") == "json_schema":
        out["response_format"] = {"type": "json_schema", "json_schema": {
            "name": fmt.get("name", "schema"), "schema": fmt.get("schema") or {}, "strict": fmt.get("strict")}}
    elif fmt.get("type") == "json_object":
        out["response_format"] = {"type": "json_object"}
    if isinstance(body.get("reasoning"), dict):
        on = body["reasoning"].get("effort") not in (None, "none", "minimal")
        out["chat_template_kwargs"] = {"enable_thinking": on, "thinking": on}
    if out["stream"]:
        out["stream_options"] = {"include_usage": True}
    return out


# ---------------------------------------------------------------------------- answer -> response object
def _usage(u: Dict[str, Any]) -> Dict[str, Any]:
    n_in, n_out = u.get("prompt_tokens", 0), u.get("completion_tokens", 0)
    cached = ((u.get("prompt_tokens_details") or {}).get("cached_tokens")) or 0
    return {"input_tokens": n_in, "input_tokens_details": {"cached_tokens": cached}, "output_tokens": n_out,
            "output_tokens_details": {"reasoning_tokens": 0}, "total_tokens": n_in + n_out}


def envelope(body: Dict[str, Any], rid: str, created: int, status: str, output: List[dict], usage=None,
             incomplete: Optional[str] = None) -> Dict[str, Any]:
    return {"id": rid, "object": "response", "created_at": created, "status": status, "error": None,
            "incomplete_details": {"reason": incomplete} if incomplete else None,
            "instructions": body.get("instructions"), "max_output_tokens": body.get("max_output_tokens"),
            "model": body.get("model", "default_model_name"), "output": output,
            "parallel_tool_calls": body.get("parallel_tool_calls", True), "temperature": body.get("temperature", 1.0),
            "top_p": body.get("top_p", 1.0), "tool_choice": body.get("tool_choice", "auto"),
            "tools": body.get("tools") or [], "text": body.get("text") or {"format": {"type": "text"}},
            "usage": _usage(usage) if usage else None, "metadata": body.get("metadata") or {}}


def _reasoning_item(text: str, status="completed") -> dict:
    return {"type": "reasoning", "id": f"rs_{uuid.uuid4().hex[:24]}", "status": status,
            "summary": [{"type": "summary_text", "text": text}]}


def _message_item(text: str, status="completed") -> dict:
    return {"type": "message", "id": f"msg_{uuid.uuid4().hex[:24]}", "role": "assistant", "status": status,
            "content": [{"type": "output_text", "text": text, "annotations": []}]}


def _call_item(call_id: str, name: str, arguments: str, status="completed") -> dict:
    return {"type": "function_call", "id": f"fc_{uuid.uuid4().hex[:24]}", "call_id": call_id, "name": name,
            "arguments": arguments, "status": status}


def chat_response_to_response(resp: Dict[str, Any], body: Dict[str, Any], rid: Optional[str] = None) -> Dict[str, Any]:
    choice = (resp.get("choices") or [{}])[0]
    msg = choice.get("message") or {}
    out: List[dict] = []
    if msg.get("reasoning_content"):
        out.append(_reasoning_item(msg["reasoning_content"]))
    if msg.get("content") or not msg.get("tool_calls"):
        out.append(_message_item(msg.get("content") or ""))
    for c in msg.get("tool_calls") or []:
        f = c.get("function") or {}
        out.append(_call_item(c.get("id") or f"call_{uuid.uuid4().hex[:24]}", f.get("name"), f.get("arguments") or "{}"))
    cut = choice.get("finish_reason") == "length"
    if cut:
        for it in out:
            if it["type"] == "message":
                it["status"] = "incomplete"
    return envelope(body, rid or f"resp_{uuid.uuid4().hex}", int(resp.get("created") or time.time()),
                    "incomplete" if cut else "completed", out, resp.get("usage") or {},
                    "max_output_tokens" if cut else None)


# ---------------------------------------------------------------------------- chat stream -> event stream
async def chat_chunks_to_events(chunks: AsyncIterator[Dict[str, Any]], body: Dict[str, Any],
                                rid: Optional[str] = None) -> AsyncIterator[bytes]:
    rid = rid or f"resp_{uuid.uuid4().hex}"
    created = int(time.time())
    seq = 0

    def ev(kind: str, **data) -> bytes:
        nonlocal seq
        d = {"type": kind, "sequence_number": seq, **data}
        seq += 1
        return f"event: {kind}\ndata: {json.dumps(d, ensure_ascii=False)}\n\n".encode()

    output: List[dict] = []
    cur: Optional[dict] = None          # the open output item
    cur_key = None                      # "reasoning" | "message" | ("call", index)
    finish, usage = None, {}

    def close():
        nonlocal cur, cur_key
        out = []
        if cur is None:
            return out
        i = len(output) - 1
        if cur["type"] == "reasoning":
            text = cur["summary"][0]["text"]
            out.append(ev("response.reasoning_summary_text.done", item_id=cur["id"], output_index=i, summary_index=0,
                          text=text))
            out.append(ev("response.reasoning_summary_part.done", item_id=cur["id"], output_index=i, summary_index=0,
                          part=cur["summary"][0]))
        elif cur["type"] == "message":
            part = cur["content"][0]
            out.append(ev("response.output_text.done", item_id=cur["id"], output_index=i, content_index=0,
                          text=part["text"]))
            out.append(ev("response.content_part.done", item_id=cur["id"], output_index=i, content_index=0, part=part))
        else:
            out.append(ev("response.function_call_arguments.done", item_id=cur["id"], output_index=i,
                          arguments=cur["arguments"]))
        cur["status"] = "completed"
        out.append(ev("response.output_item.done", output_index=i, item=cur))
        cur = cur_key = None
        return out

    def open_item(key, item):
        nonlocal cur, cur_key
        out = close()
        cur, cur_key = item, key
        output.append(item)
        i = len(output) - 1
        out.append(ev("response.output_item.added", output_index=i, item=json.loads(json.dumps(item))))
        if item["type"] == "reasoning":
            out.append(ev("response.reasoning_summary_part.added", item_id=item["id"], output_index=i, summary_index=0,
                          part={"type": "summary_text", "text": ""}))
        elif item["type"] == "message":
            out.append(ev("response.content_part.added", item_id=item["id"], output_index=i, content_index=0,
                          part={"type": "output_text", "text": "", "annotations": []}))
        return out

    yield ev("response.created", response=envelope(body, rid, created, "in_progress", []))
    yield ev("response.in_progress", response=envelope(body, rid, created, "in_progress", []))
    async for chunk in chunks:
        if chunk.get("usage"):
            usage = chunk["usage"]
        for choice in chunk.get("choices") or []:
            delta = choice.get("delta") or {}
            if delta.get("reasoning_content"):
                if cur_key != "reasoning":
                    for e in open_item("reasoning", _reasoning_item("", "in_progress")):
                        yield e
                cur["summary"][0]["text"] += delta["reasoning_content"]
                yield ev("response.reasoning_summary_text.delta", item_id=cur["id"], output_index=len(output) - 1,
                         summary_index=0, delta=delta["reasoning_content"])
            if delta.get("content"):
                if cur_key != "message":
                    for e in open_item("message", _message_item("", "in_progress")):
                        yield e
                cur["content"][0]["text"] += delta["content"]
                yield ev("response.output_text.delta", item_id=cur["id"], output_index=len(output) - 1,
                         content_index=0, delta=delta["content"])
            for c in delta.get("tool_calls") or []:
                f = c.get("function") or {}
                key = ("call", c.get("index", 0))
                if f.get("name") or cur_key != key:
                    for e in open_item(key, _call_item(c.get("id") or f"call_{uuid.uuid4().hex[:24]}",
                                                       f.get("name") or "", "", "in_progress")):
                        yield e
                if f.get("arguments"):
                    cur["arguments"] += f["arguments"]
                    yield ev("response.function_call_arguments.delta", item_id=cur["id"],
                             output_index=len(output) - 1, delta=f["arguments"])
            if choice.get("finish_reason"):
                finish = choice["finish_reason"]
    if not output:
        for e in open_item("message", _message_item("", "in_progress")):
            yield e
    for e in close():
        yield e
    cut = finish == "length"
    final = envelope(body, rid, created, "incomplete" if cut else "completed", output, usage,
                     "max_output_tokens" if cut else None)
    yield ev("response.incomplete" if cut else "response.completed", response=final)


# ---------------------------------------------------------------------------- route
async def responses_impl(raw: Request, g):
    from .api_models import ChatCompletionRequest
    from .api_openai import chat_completions_impl, create_error_response

    try:
        body = await raw.json()
    except ValueError:
        return create_error_response(400, "the request body is not JSON")
    if body.get("input") in (None, "", []):
        return create_error_response(400, "input: a string or a list of items is required")
    body.setdefault("model", g.args.model_name)
    try:
        request = ChatCompletionRequest(**to_chat_request(body))
    except Exception as e:
        return create_error_response(400, f"invalid request: {e}")
    resp = await chat_completions_impl(request, raw, g)
    rid = f"resp_{uuid.uuid4().hex}"
    if getattr(resp, "body_iterator", None) is not None:
        if resp.status_code != 200:
            return resp
        return await stream_response(chat_chunks_to_events(sse_to_chunks(resp.body_iterator), body, rid), g)
    if resp.status_code != 200:
        return resp
    return JSONResponse(chat_response_to_response(json.loads(bytes(resp.body)), body, rid))
