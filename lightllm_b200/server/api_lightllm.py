"""Native routes: /generate, /generate_stream, /get_score.
Request:  {"inputs": str | [int], "parameters": {...sampling params, "return_details"?}, "multimodal_params"?}
Response: {"generated_text": [...], "count_output_tokens", "finish_reason", "prompt_tokens", "logprobs", ["tokens"]}
Stream:   SSE lines  data:{"token": {...}, "generated_text": null, "finished": bool, "finish_reason": ..., "details": null}
Reference: lightllm/server/api_lightllm.py:12-170.
"""
from __future__ import annotations

import json
from collections import defaultdict

from fastapi import Request
from .api_stream_obj import stream_response
from fastapi.responses import JSONResponse, Response, StreamingResponse

from .core.objs.sampling_params import SamplingParams


def _make_params(g, params: dict) -> SamplingParams:
    sp = SamplingParams()
    sp.init(tokenizer=g.httpserver_manager.tokenizer, **params)
    sp.verify(g.args.vocab_size)
    return sp


async def lightllm_get_score(request: Request, g) -> Response:
    body = await request.json()
    prompt = body.pop("chat", None) or body.pop("inputs")
    params = body.get("parameters", {})
    params["max_new_tokens"] = 1
    sp = _make_params(g, params)
    score, prompt_tokens = None, 0
    async for sub_id, text, meta, fs in g.httpserver_manager.generate(prompt, sp, body.get("multimodal_params"), request):
        prompt_tokens = meta.get("prompt_tokens", 0)
        score = meta.get("score")
    if score is None:
        st = None
    return JSONResponse({"score": score, "prompt_tokens": prompt_tokens, "finish_reason": "stop"})


async def lightllm_generate(request: Request, g) -> Response:
    body = await request.json()
    prompt = body.pop("inputs")
    params = dict(body.pop("parameters", {}))
    return_details = params.pop("return_details", False)
    prompt_lp = input_usage = None
    return_routed = params.pop("return_routed_experts", bool(getattr(g.args, "enable_return_routed_experts", False)))
    routed = {}
    sp = _make_params(g, params)
    mm = body.get("multimodal_params")
    texts = defaultdict(list)
    tokens = defaultdict(list)
    count = defaultdict(int)
    finish = {}
    logprobs = defaultdict(list)
    prompt_tokens = 0
    async for sub_id, text, meta, fs in g.httpserver_manager.generate(prompt, sp, mm, request):
        count[sub_id] += 1
        texts[sub_id].append(text)
        logprobs[sub_id].append(meta.get("logprob"))
        prompt_tokens = meta.get("prompt_tokens", prompt_tokens)
        if "routed_experts" in meta:     # travels with the last token only; kept out of the per-token details
            routed[sub_id] = meta.pop("routed_experts")
        if "input_usage" in meta:
            input_usage = meta.pop("input_usage")
        if "prompt_logprobs" in meta:
            prompt_lp = (meta.pop("prompt_token_ids", None), meta.pop("prompt_logprobs"))
        if return_details:
            m = dict(meta)
            m["text"] = text
            tokens[sub_id].append(m)
        if fs.is_finished():
            finish[sub_id] = fs.get_finish_reason()
    ids = sorted(texts)
    ret = {"generated_text": ["".join(texts[i]) for i in ids],
           "count_output_tokens": count[ids[0]] if len(ids) == 1 else [count[i] for i in ids],
           "finish_reason": finish.get(ids[0]) if len(ids) == 1 else [finish.get(i) for i in ids],
           "prompt_tokens": prompt_tokens,
           "logprobs": logprobs[ids[0]] if len(ids) == 1 else [logprobs[i] for i in ids]}
    if return_details:
        ret["tokens"] = tokens[ids[0]] if len(ids) == 1 else [tokens[i] for i in ids]
    if prompt_lp is not None:
        ret["prompt_token_ids"], ret["prompt_logprobs"] = prompt_lp
    if input_usage is not None:
        ret["input_usage"] = input_usage
    if return_routed and routed:
        ret["routed_experts"] = routed.get(ids[0]) if len(ids) == 1 else [routed.get(i) for i in ids]
    return Response(content=json.dumps(ret, ensure_ascii=False).encode("utf-8"), media_type="application/json")


async def lightllm_generate_stream(request: Request, g) -> Response:
    body = await request.json()
    prompt = body.pop("inputs")
    params = dict(body.pop("parameters", {}))
    params.pop("return_details", None)
    sp = _make_params(g, params)
    if sp.best_of != 1:
        raise ValueError("streaming needs best_of == 1")
    mm = body.get("multimodal_params")
    gen = g.httpserver_manager.generate(prompt, sp, mm, request)

    async def stream():
        async for sub_id, text, meta, fs in gen:
            ret = {"token": {"id": meta.get("id"), "text": text, "logprob": meta.get("logprob"),
                             "special": meta.get("special", False), "count_output_tokens": meta.get("count_output_tokens"),
                             "prompt_tokens": meta.get("prompt_tokens")},
                   "generated_text": None, "finished": fs.is_finished(), "finish_reason": fs.get_finish_reason(),
                   "details": None}
            yield ("data:" + json.dumps(ret, ensure_ascii=False) + "\n\n").encode("utf-8")

    return await stream_response(stream(), g)
