"""OpenAI-compatible routes: /v1/chat/completions and /v1/completions (streaming and not), with
tool-call and reasoning-content post-processing.  Parameter mapping follows the reference
(lightllm/server/api_openai.py:292-360): n -> n/best_of, max_completion_tokens | max_tokens ->
max_new_tokens, stop -> stop_sequences, response_format -> guided_json / guided_grammar, and the
template already adds special tokens (add_special_tokens=False).
"""
from __future__ import annotations

import json
import time
import uuid
from typing import AsyncGenerator, Dict, List

from fastapi import Request
from .api_stream_obj import stream_response
from fastapi.responses import JSONResponse, Response, StreamingResponse

from .api_models import (ChatCompletionRequest, ChatCompletionResponse, ChatCompletionResponseChoice,
                         ChatCompletionStreamResponse, ChatCompletionStreamResponseChoice, ChatMessage,
                         CompletionChoice, CompletionLogprobs, CompletionRequest, CompletionResponse,
                         CompletionStreamChoice, CompletionStreamResponse, DeltaMessage, FunctionResponse,
                         PromptTokensDetails, ToolCall, UsageInfo)
from .build_prompt import build_prompt
from .core.objs.sampling_params import SamplingParams
from .function_call_parser import FunctionCallParser
from .reasoning_parser import ReasoningParser


def create_error_response(status_code: int, message: str, err_type: str = "invalid_request_error") -> JSONResponse:
    return JSONResponse({"error": {"message": message, "type": err_type, "param": None, "code": status_code}},
                        status_code=status_code)


def _sampling_dict(req, max_new: int, stop, n: int) -> dict:
    d = {"do_sample": req.do_sample, "presence_penalty": req.presence_penalty,
         "frequency_penalty": req.frequency_penalty, "repetition_penalty": req.repetition_penalty,
         "temperature": req.temperature, "top_p": req.top_p, "top_k": req.top_k, "ignore_eos": req.ignore_eos,
         "max_new_tokens": max_new, "stop_sequences": stop, "n": n, "best_of": n, "add_special_tokens": False,
         "seed": req.seed, "min_new_tokens": req.min_new_tokens}
    rf = getattr(req, "response_format", None)
    if rf is not None:
        if rf.type == "json_schema" and rf.json_schema is not None and rf.json_schema.schema_ is not None:
            d["guided_json"] = rf.json_schema.schema_
        elif rf.type == "json_object":
            d["guided_grammar"] = "json"
    if getattr(req, "guided_regex", None):
        d["regular_constraint"] = req.guided_regex
    elif getattr(req, "guided_grammar", None) and "guided_grammar" not in d and "guided_json" not in d:
        d["guided_grammar"] = req.guided_grammar
    return d


def _usage(prompt_tokens: int, completion_tokens: int, cached: int) -> UsageInfo:
    return UsageInfo(prompt_tokens=prompt_tokens, completion_tokens=completion_tokens,
                     total_tokens=prompt_tokens + completion_tokens,
                     prompt_tokens_details=PromptTokensDetails(cached_tokens=cached))


async def chat_completions_impl(request: ChatCompletionRequest, raw_request: Request, g) -> Response:
    if request.logit_bias is not None:
        return create_error_response(400, "The logit_bias parameter is not currently supported")
    if request.function_call is not None and request.function_call != "none":
        return create_error_response(400, "The function call feature is not supported")
    created = int(time.time())
    tools = None
    if request.tools and request.tool_choice != "none":
        tools = [t.function.model_dump() for t in request.tools]
        if not isinstance(request.tool_choice, str):
            tools = [t for t in tools if t["name"] == request.tool_choice.function.name]
    prompt = await build_prompt(request, tools)
    max_new = request.max_completion_tokens or request.max_tokens or 65536
    sp = SamplingParams()
    sp.init(tokenizer=g.httpserver_manager.tokenizer, **_sampling_dict(request, max_new, request.stop, request.n))
    sp.verify(g.args.vocab_size)
    gen = g.httpserver_manager.generate(prompt, sp, None, raw_request)
    req_id = f"chatcmpl-{uuid.uuid4().hex}"
    tool_parser_name = g.args.tool_call_parser
    reasoning_name = g.args.reasoning_parser

    if not request.stream:
        texts: Dict[int, List[str]] = {}
        lps: Dict[int, list] = {}
        finish: Dict[int, str] = {}
        prompt_tokens, cached = 0, 0
        counts: Dict[int, int] = {}
        async for sub_id, text, meta, fs in gen:
            texts.setdefault(sub_id, []).append(text)
            lps.setdefault(sub_id, []).append((text, meta.get("logprob")))
            counts[sub_id] = counts.get(sub_id, 0) + 1
            prompt_tokens = meta.get("prompt_tokens", prompt_tokens)
            cached = meta.get("prompt_cache_len", cached)
            if fs.is_finished():
                finish[sub_id] = fs.get_finish_reason()
        choices = []
        for i, sid in enumerate(sorted(texts)):
            full = "".join(texts[sid])
            reasoning = None
            if reasoning_name and request.separate_reasoning:
                reasoning, full = ReasoningParser(reasoning_name, stream_reasoning=False).parse_non_stream(full)
            tool_calls = None
            reason = finish.get(sid)
            if tools and tool_parser_name:
                parser = FunctionCallParser(request.tools, tool_parser_name)
                if parser.has_tool_call(full):
                    full, calls = parser.parse_non_stream(full)
                    tool_calls = [ToolCall(id=f"call_{uuid.uuid4().hex[:24]}", index=getattr(c, "tool_index", j),
                                           function=FunctionResponse(name=c.name, arguments=c.parameters))
                                  for j, c in enumerate(calls)]
                    if tool_calls and reason == "stop":
                        reason = "tool_calls"
            logprobs = None
            if request.logprobs:
                logprobs = {"content": [{"token": t, "logprob": lp, "bytes": list(t.encode()), "top_logprobs": []}
                                        for t, lp in lps[sid]]}
            choices.append(ChatCompletionResponseChoice(
                index=i, message=ChatMessage(role="assistant", content=full, reasoning_content=reasoning,
                                             tool_calls=tool_calls), logprobs=logprobs, finish_reason=reason))
        total_out = sum(counts.values())
        resp = ChatCompletionResponse(id=req_id, created=created, model=request.model, choices=choices,
                                      usage=_usage(prompt_tokens, total_out, cached))
        return JSONResponse(resp.model_dump(exclude_none=False))

    if request.n != 1:
        return create_error_response(400, "streaming needs n == 1")

    async def stream() -> AsyncGenerator[bytes, None]:
        parser = FunctionCallParser(request.tools, tool_parser_name) if (tools and tool_parser_name) else None
        reasoner = ReasoningParser(reasoning_name, stream_reasoning=request.stream_reasoning) \
            if (reasoning_name and request.separate_reasoning) else None
        first = True
        out_tokens, prompt_tokens, cached = 0, 0, 0
        saw_tool = False
        async for sub_id, text, meta, fs in gen:
            out_tokens += 1
            prompt_tokens = meta.get("prompt_tokens", prompt_tokens)
            cached = meta.get("prompt_cache_len", cached)
            delta_kwargs = {}
            if first:
                delta_kwargs["role"] = "assistant"
                first = False
            reasoning_piece = None
            if reasoner is not None:
                reasoning_piece, text = reasoner.parse_stream_chunk(text)
            tool_deltas = None
            if parser is not None:
                text, calls = parser.parse_stream_chunk(text)
                if calls:
                    saw_tool = True
                    tool_deltas = [ToolCall(id=f"call_{uuid.uuid4().hex[:24]}" if c.name else None, index=c.tool_index,
                                            function=FunctionResponse(name=c.name, arguments=c.parameters)) for c in calls]
            reason = fs.get_finish_reason() if fs.is_finished() else None
            if reason == "stop" and saw_tool:
                reason = "tool_calls"
            lp = None
            if request.logprobs:
                lp = {"content": [{"token": text, "logprob": meta.get("logprob"), "bytes": list(text.encode()),
                                   "top_logprobs": []}]}
            choice = ChatCompletionStreamResponseChoice(
                index=0, delta=DeltaMessage(content=text or ("" if not (reasoning_piece or tool_deltas) else None),
                                            reasoning_content=reasoning_piece, tool_calls=tool_deltas, **delta_kwargs),
                logprobs=lp, finish_reason=reason)
            chunk = ChatCompletionStreamResponse(id=req_id, created=created, model=request.model, choices=[choice])
            yield ("data: " + json.dumps(chunk.model_dump(exclude_none=True), ensure_ascii=False) + "\n\n").encode()
        if request.stream_options and request.stream_options.include_usage:
            chunk = ChatCompletionStreamResponse(id=req_id, created=created, model=request.model, choices=[],
                                                 usage=_usage(prompt_tokens, out_tokens, cached))
            yield ("data: " + json.dumps(chunk.model_dump(exclude_none=True), ensure_ascii=False) + "\n\n").encode()
        yield b"data: [DONE]\n\n"

    return await stream_response(stream(), g)


def _completion_logprobs(tokenizer, out_tokens, out_lps, prompt_ids, prompt_lp, drop_output: bool):
    """`logprobs` of a completion choice: with echo the prompt's tokens first (logprob None for the first one), each
    with its own logprob and, when the engine computed them, the most likely tokens at that position."""
    tokens, token_lps, tops, offsets = [], [], [], []
    off = 0

    def push(text, lp, top):
        nonlocal off
        tokens.append(text)
        token_lps.append(lp)
        tops.append(top)
        offsets.append(off)
        off += len(text)

    if prompt_ids is not None:
        for pos, tid in enumerate(prompt_ids):
            try:
                text = tokenizer.decode([tid], skip_special_tokens=False)
            except Exception:
                text = f"<{tid}>"
            entry = prompt_lp[pos] if (prompt_lp is not None and pos < len(prompt_lp)) else None
            if not entry:
                push(text, None, None)
                continue
            own = entry.get(tid) or entry.get(str(tid)) or {}
            top = {(v.get("decoded_token") or str(k)): v["logprob"] for k, v in entry.items()}
            push(text, own.get("logprob"), top)
    if not drop_output:
        for text, lp in zip(out_tokens, out_lps):
            push(text, lp, {text: lp} if lp is not None else None)
    return CompletionLogprobs(tokens=tokens, token_logprobs=token_lps, top_logprobs=tops, text_offset=offsets)


async def completions_impl(request: CompletionRequest, raw_request: Request, g) -> Response:
    if request.logit_bias is not None:
        return create_error_response(400, "The logit_bias parameter is not currently supported")
    created = int(time.time())
    prompts = request.prompt
    if isinstance(prompts, str) or (isinstance(prompts, list) and prompts and isinstance(prompts[0], int)):
        prompts = [prompts]
    if request.stream and len(prompts) != 1:
        return create_error_response(400, "streaming needs a single prompt")
    n = max(request.n or 1, request.best_of or 1)
    max_new = request.max_tokens if request.max_tokens is not None else 16
    req_id = f"cmpl-{uuid.uuid4().hex}"
    mgr = g.httpserver_manager

    # echo + logprobs: the prompt's own token logprobs come back too (what evaluation harnesses score continuations
    # with); needs --enable_prompt_logprobs, otherwise the prompt tokens are echoed without logprobs
    want_prompt_lp = bool(request.echo and request.logprobs is not None and
                          getattr(g.args, "enable_prompt_logprobs", False) and not request.stream)

    def make_sp():
        sp = SamplingParams()
        d = _sampling_dict(request, max(max_new, 1), request.stop, n)
        d["add_special_tokens"] = True
        if want_prompt_lp:
            d["prompt_logprobs"] = max(0, min(int(request.logprobs), 20))
        sp.init(tokenizer=mgr.tokenizer, **d)
        sp.verify(g.args.vocab_size)
        return sp

    if request.stream:
        gen = mgr.generate(prompts[0], make_sp(), None, raw_request)

        async def stream():
            out_tokens, prompt_tokens, cached = 0, 0, 0
            async for sub_id, text, meta, fs in gen:
                out_tokens += 1
                prompt_tokens = meta.get("prompt_tokens", prompt_tokens)
                cached = meta.get("prompt_cache_len", cached)
                lp = None
                if request.logprobs is not None:
                    lp = {"tokens": [text], "token_logprobs": [meta.get("logprob")], "top_logprobs": [], "text_offset": []}
                ch = CompletionStreamChoice(text=text, index=0, logprobs=lp,
                                            finish_reason=fs.get_finish_reason() if fs.is_finished() else None)
                chunk = CompletionStreamResponse(id=req_id, created=created, model=request.model, choices=[ch])
                yield ("data: " + json.dumps(chunk.model_dump(exclude_none=True), ensure_ascii=False) + "\n\n").encode()
            if request.stream_options and request.stream_options.include_usage:
                chunk = CompletionStreamResponse(id=req_id, created=created, model=request.model, choices=[],
                                                 usage=_usage(prompt_tokens, out_tokens, cached))
                yield ("data: " + json.dumps(chunk.model_dump(exclude_none=True), ensure_ascii=False) + "\n\n").encode()
            yield b"data: [DONE]\n\n"

        return await stream_response(stream(), g)

    choices = []
    total_prompt, total_out, cached = 0, 0, 0
    for pi, prompt in enumerate(prompts):
        texts: Dict[int, list] = {}
        lps: Dict[int, list] = {}
        finish: Dict[int, str] = {}
        ptoks = 0
        prompt_lp = prompt_ids = None
        async for sub_id, text, meta, fs in mgr.generate(prompt, make_sp(), None, raw_request):
            if "prompt_logprobs" in meta:
                prompt_lp, prompt_ids = meta.pop("prompt_logprobs"), meta.pop("prompt_token_ids", None)
            texts.setdefault(sub_id, []).append(text)
            lps.setdefault(sub_id, []).append(meta.get("logprob"))
            ptoks = meta.get("prompt_tokens", ptoks)
            cached = max(cached, meta.get("prompt_cache_len", 0))
            total_out += 1
            if fs.is_finished():
                finish[sub_id] = fs.get_finish_reason()
        total_prompt += ptoks
        for sid in sorted(texts):
            body = "".join(texts[sid])
            if request.echo and isinstance(prompt, str):
                body = prompt + body
            lp = None
            if request.logprobs is not None:
                lp = _completion_logprobs(mgr.tokenizer, texts[sid], lps[sid], prompt_ids if request.echo else None,
                                          prompt_lp, request.max_tokens == 0)
                if request.echo and prompt_ids is not None and not isinstance(prompt, str):
                    body = "".join(lp.tokens[: len(prompt_ids)]) + body
            if request.max_tokens == 0:       # scoring only: nothing of the one token the engine produced is shown
                total_out -= len(texts[sid])
                body = prompt if (request.echo and isinstance(prompt, str)) else \
                    ("".join(lp.tokens) if (lp is not None and request.echo) else "")
            choices.append(CompletionChoice(text=body, index=len(choices), logprobs=lp, finish_reason=finish.get(sid)))
    resp = CompletionResponse(id=req_id, created=created, model=request.model, choices=choices,
                              usage=_usage(total_prompt, total_out, cached))
    return JSONResponse(resp.model_dump())
