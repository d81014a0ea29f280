"""TGI-compatible request/response shapes over the same generate() generator
(reference: lightllm/server/api_tgi.py)."""
from __future__ import annotations

import json
import os

from fastapi import Request
from .api_stream_obj import stream_response
from fastapi.responses import JSONResponse, Response, StreamingResponse

from .core.objs.sampling_params import SamplingParams


# `RETURN_LIST=1`: the non-streaming answer is wrapped in a list, as the hosted inference API does
RETURN_LIST = os.getenv("RETURN_LIST", "FALSE").upper() in ("ON", "TRUE", "1")


def _params(d: dict) -> dict:
    p = dict(d or {})
    out = {"max_new_tokens": p.get("max_new_tokens", 20), "do_sample": p.get("do_sample", False),
           "temperature": p.get("temperature") or 1.0, "top_p": p.get("top_p") or 1.0,
           "top_k": p.get("top_k") or -1, "repetition_penalty": p.get("repetition_penalty") or 1.0,
           "stop_sequences": p.get("stop") or p.get("stop_sequences"), "seed": p.get("seed", -1)}
    if p.get("best_of"):
        out["best_of"] = out["n"] = p["best_of"]
    return out


async def tgi_generate_impl(request: Request, g) -> Response:
    body = getattr(request, "_json", None) or await request.json()
    params = body.get("parameters") or {}
    sp = SamplingParams().init(tokenizer=g.httpserver_manager.tokenizer, **_params(params))
    sp.verify(g.args.vocab_size)
    texts, toks, finish, prompt_tokens = {}, {}, {}, 0
    async for sub_id, text, meta, fs in g.httpserver_manager.generate(body["inputs"], sp, None, request):
        texts.setdefault(sub_id, []).append(text)
        toks.setdefault(sub_id, []).append({"id": meta.get("id"), "text": text, "logprob": meta.get("logprob"),
                                            "special": meta.get("special", False)})
        prompt_tokens = meta.get("prompt_tokens", prompt_tokens)
        if fs.is_finished():
            finish[sub_id] = fs.get_finish_reason()
    first = sorted(texts)[0]
    ret = {"generated_text": "".join(texts[first])}
    if params.get("details") or params.get("return_details"):
        ret["details"] = {"finish_reason": {"stop": "eos_token", "length": "length"}.get(finish.get(first), finish.get(first)),
                          "generated_tokens": len(toks[first]), "prefill": [], "tokens": toks[first],
                          "seed": params.get("seed")}
        if len(texts) > 1:
            ret["details"]["best_of_sequences"] = [{"generated_text": "".join(texts[i]), "tokens": toks[i]}
                                                   for i in sorted(texts)[1:]]
    return JSONResponse([ret] if RETURN_LIST else ret)


async def tgi_generate_stream_impl(request: Request, g) -> Response:
    body = getattr(request, "_json", None) or await request.json()
    params = body.get("parameters") or {}
    sp = SamplingParams().init(tokenizer=g.httpserver_manager.tokenizer, **_params(params))
    sp.verify(g.args.vocab_size)
    gen = g.httpserver_manager.generate(body["inputs"], sp, None, request)

    async def stream():
        all_text = []
        async for sub_id, text, meta, fs in gen:
            all_text.append(text)
            ret = {"token": {"id": meta.get("id"), "text": text, "logprob": meta.get("logprob"),
                             "special": meta.get("special", False)},
                   "generated_text": "".join(all_text) if fs.is_finished() else None,
                   "details": {"finish_reason": fs.get_finish_reason(), "generated_tokens": len(all_text)}
                   if fs.is_finished() else None}
            yield ("data:" + json.dumps(ret, ensure_ascii=False) + "\n\n").encode()

    return await stream_response(stream(), g)
