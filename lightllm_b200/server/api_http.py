"""FastAPI application served by every HTTP worker.

Routes (same surface as the reference, lightllm/server/api_http.py:173-544): liveness/readiness,
/get_model_name, /get_server_info, /get_weight_version, /health(z), /token_load, /generate,
/generate_stream, /get_score, / (TGI-compatible), /v1/chat/completions, /v1/completions,
/v1/models, /tokens, /metrics, /profiler_start|stop, plus the RL control routes when enabled.
Errors: client disconnect 499, ServerBusyError 429, bad parameters 400, anything else 417.
"""
from __future__ import annotations

import asyncio
import json
import os
import time
from dataclasses import dataclass
from typing import Optional

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, Response

from ..utils.errors import ServerBusyError
from ..utils.health_check import health_check
from .api_models import ChatCompletionRequest, CompletionRequest, ModelCard, ModelListResponse
from .core.objs.sampling_params import ParamError, SamplingParams
from .core.objs.start_args import StartArgs, get_env_start_args


@dataclass
class G_Objs:
    app: Optional[FastAPI] = None
    args: Optional[StartArgs] = None
    httpserver_manager = None
    metric_client = None
    token_load = None
    g_generate_func = None
    g_generate_stream_func = None

    def set_args(self, args: StartArgs):
        from .api_lightllm import lightllm_generate, lightllm_generate_stream
        from .api_tgi import tgi_generate_impl, tgi_generate_stream_impl
        from .build_prompt import init_tokenizer
        from .router.token_load import TokenLoad

        self.args = args
        if args.use_tgi_api:
            self.g_generate_func, self.g_generate_stream_func = tgi_generate_impl, tgi_generate_stream_impl
        else:
            self.g_generate_func, self.g_generate_stream_func = lightllm_generate, lightllm_generate_stream
        if args.metric_port:
            from .metrics.manager import MetricClient

            self.metric_client = MetricClient(args)
        if args.run_mode == "pd_master":
            from .httpserver_for_pd_master.manager import HttpServerManagerForPDMaster

            self.httpserver_manager = HttpServerManagerForPDMaster(args, self.metric_client)
        else:
            from .httpserver.manager import HttpServerManager

            self.httpserver_manager = HttpServerManager(args, self.metric_client)
            SamplingParams.load_generation_cfg(args.model_dir)
            init_tokenizer(self.httpserver_manager.tokenizer, args.chat_template)
            self.token_load = TokenLoad(f"{args.unique_server_name}_token_load", max(1, args.dp // args.nnodes))


g_objs = G_Objs()
app = FastAPI()
g_objs.app = app


@app.middleware("http")
async def echo_request_id(request: Request, call_next):
    """A caller's X-Request-Id comes back on the response, so that proxies and clients can pair the two."""
    response = await call_next(request)
    xid = request.headers.get("X-Request-Id")
    if xid:
        response.headers["X-Request-Id"] = xid
    return response


def create_error_response(status_code: int, message: str) -> JSONResponse:
    if g_objs.metric_client is not None:
        g_objs.metric_client.counter_inc("lightllm_request_failure")
    return JSONResponse({"message": message}, status_code=status_code)


async def _guard(coro):
    try:
        return await coro
    except ServerBusyError as e:
        return create_error_response(429, str(e))
    except (ParamError, ValueError, KeyError, json.JSONDecodeError) as e:
        return create_error_response(400, f"{type(e).__name__}: {e}")
    except asyncio.CancelledError as e:
        return create_error_response(499, str(e) or "client disconnected")
    except Exception as e:
        return create_error_response(417, f"{type(e).__name__}: {e}")


@app.get("/liveness")
@app.post("/liveness")
def liveness():
    return {"status": "ok"}


@app.get("/readiness")
@app.post("/readiness")
def readiness():
    return {"status": "ok"}


@app.get("/get_model_name")
@app.post("/get_model_name")
def get_model_name():
    return {"model_name": g_objs.args.model_name}


@app.get("/get_server_info")
@app.post("/get_server_info")
def get_server_info():
    d = {k: v for k, v in g_objs.args.to_dict().items() if not k.startswith("_")}
    return JSONResponse(json.loads(json.dumps(d, default=str)))


@app.get("/get_weight_version")
@app.post("/get_weight_version")
def get_weight_version():
    return {"weight_version": g_objs.args.weight_version}


def _mk_sp(d):
    sp = SamplingParams()
    sp.init(tokenizer=None, **d)
    return sp


@app.get("/healthz")
@app.get("/health")
@app.head("/health")
async def healthcheck(request: Request):
    ok = await health_check(g_objs.httpserver_manager, _mk_sp)
    return JSONResponse({"message": "Ok" if ok else "Error"}, status_code=200 if ok else 503)


@app.get("/token_load")
async def token_load(request: Request):
    snap = g_objs.token_load.snapshot() if g_objs.token_load is not None else []
    if len(snap) == 1:
        return JSONResponse(snap[0])
    return JSONResponse(snap)


@app.post("/generate")
async def generate(request: Request) -> Response:
    return await _guard(g_objs.g_generate_func(request, g_objs))


@app.post("/generate_stream")
async def generate_stream(request: Request) -> Response:
    return await _guard(g_objs.g_generate_stream_func(request, g_objs))


@app.post("/get_score")
async def get_score(request: Request) -> Response:
    from .api_lightllm import lightllm_get_score

    return await _guard(lightllm_get_score(request, g_objs))


@app.post("/")
async def compat_generate(request: Request) -> Response:
    body = await request.json()
    request._json = body
    if body.get("stream", False):
        return await generate_stream(request)
    return await generate(request)


@app.post("/v1/chat/completions")
async def chat_completions(request: ChatCompletionRequest, raw_request: Request) -> Response:
    from .api_openai import chat_completions_impl

    return await _guard(chat_completions_impl(request, raw_request, g_objs))


@app.post("/v1/completions")
async def completions(request: CompletionRequest, raw_request: Request) -> Response:
    from .api_openai import completions_impl

    return await _guard(completions_impl(request, raw_request, g_objs))


@app.post("/v1/messages")
async def anthropic_messages(raw_request: Request) -> Response:
    from .api_anthropic import anthropic_messages_impl

    return await _guard(anthropic_messages_impl(raw_request, g_objs))


@app.post("/v1/messages/count_tokens")
async def anthropic_count_tokens(raw_request: Request) -> Response:
    from .api_anthropic import anthropic_count_tokens_impl

    return await _guard(anthropic_count_tokens_impl(raw_request, g_objs))


@app.post("/v1/responses")
async def openai_responses(raw_request: Request) -> Response:
    from .api_responses import responses_impl

    return await _guard(responses_impl(raw_request, g_objs))


@app.get("/v1/models", response_model=ModelListResponse)
@app.post("/v1/models", response_model=ModelListResponse)
async def get_models(request: Request):
    a = g_objs.args
    return ModelListResponse(data=[ModelCard(id=a.model_name, owned_by=a.model_owner or "lightllm_b200",
                                             max_model_len=a.max_req_total_len)])


@app.get("/tokens")
@app.post("/tokens")
async def tokens(request: Request):
    try:
        body = await request.json()
        text = body.pop("text")
        params = body.get("parameters") or {}
        n = g_objs.httpserver_manager.tokens(text, body.get("multimodal_params"), None, params)
        return JSONResponse({"ntokens": n})
    except Exception as e:
        return create_error_response(417, f"error: {e}")


@app.get("/metrics")
async def metrics() -> Response:
    data = g_objs.metric_client.generate_latest() if g_objs.metric_client is not None else b""
    return Response(data, media_type="text/plain")


@app.get("/profiler_start")
@app.post("/profiler_start")
async def profiler_start():
    if not g_objs.args.enable_profiling:
        return create_error_response(400, "start the server with --enable_profiling")
    await g_objs.httpserver_manager.profiler_cmd("start")
    return {"status": "ok"}


@app.get("/profiler_stop")
@app.post("/profiler_stop")
async def profiler_stop():
    if not g_objs.args.enable_profiling:
        return create_error_response(400, "start the server with --enable_profiling")
    await g_objs.httpserver_manager.profiler_cmd("stop")
    return {"status": "ok"}


@app.on_event("shutdown")
async def shutdown():
    pass


@app.on_event("startup")
async def startup_event():
    args = get_env_start_args()
    g_objs.set_args(args)
    if args.enable_rl:
        from .api_http_rl import add_rl_routes

        add_rl_routes(app, g_objs)
    if args.run_mode in ("prefill", "decode", "pd_master"):
        from .api_http_pd import add_pd_routes

        add_pd_routes(app, g_objs)
    loop = asyncio.get_event_loop()
    loop.create_task(g_objs.httpserver_manager.handle_loop())
    from .httpserver import multinode_relay

    if multinode_relay.enabled(args):
        if args.node_rank == 0:
            relay = multinode_relay.RelayMaster(args.multinode_httpmanager_port, args.nnodes - 1,
                                                key=multinode_relay.relay_key(args))
            await relay.wait_peers()
            g_objs.httpserver_manager.relay_master = relay
        else:
            relay = multinode_relay.RelayFollower(args.nccl_host, args.multinode_httpmanager_port, args.node_rank,
                                                  key=multinode_relay.relay_key(args))
            await relay.hello()
            g_objs.relay_task = loop.create_task(relay.follow(g_objs.httpserver_manager))
    if args.run_mode == "pd_master" and getattr(args, "config_server_host", None) and args.config_server_port:
        g_objs.pd_master_register_task = loop.create_task(g_objs.httpserver_manager.keep_registered_at_config_server())
    if args.run_mode in ("prefill", "decode"):
        from .httpserver.pd_loop import start_pd_loops

        g_objs.pd_tasks = start_pd_loops(g_objs)
