"""Argument normalisation and process start-up.

`normalize_args` fills the derived values the same way the reference launcher does
(lightllm/server/api_start.py:36-399): max_req_total_len from the model config, router_token_ratio
0.85 (0.0 on prefill/decode nodes), batch_max_tokens = 16384 / dp, chunked_prefill_size = half of
it, eos ids and dtype from config.json, a unique name that namespaces every shm segment and ipc
socket so several servers can share a host, and the mode compatibility checks.  Start order:
metric manager -> detokenizer -> router (which spawns one model process per GPU) -> HTTP workers.
"""
from __future__ import annotations

import os
import sys
import time
import uuid

from ..utils import config_utils
from ..utils.net_utils import alloc_can_use_network_port, require_free_ports
from ..utils.process_utils import process_manager, set_proc_title
from .core.objs.start_args import StartArgs, set_env_start_args


def normalize_args(args: StartArgs, config_override: dict = None) -> StartArgs:
    a = args
    from .api_cli import compat_only_flags_in_use

    ignored = compat_only_flags_in_use(a)
    if ignored:
        print("[lightllm_b200] accepted for compatibility, without effect here: " +
              ", ".join("--" + n for n in ignored), flush=True)
    assert a.tp >= 1 and a.dp >= 1 and a.tp % a.dp == 0, "--dp must divide --tp"
    assert a.tp % a.nnodes == 0, "--tp must be a multiple of --nnodes"
    if a.run_mode in ("normal", "prefill", "decode", "visual_only"):
        assert a.model_dir is not None or config_override is not None, "--model_dir is required"
    cfg = config_override
    # ---- model-derived ----
    if a.max_req_total_len is None:
        a.max_req_total_len = config_utils.get_model_max_len(a.model_dir) if cfg is None else \
            cfg.get("max_position_embeddings", 16384)
    if a.eos_id is None:
        a.eos_ids = (config_utils.get_eos_token_ids(a.model_dir) if cfg is None else
                     ([cfg["eos_token_id"]] if isinstance(cfg.get("eos_token_id"), int) else list(cfg.get("eos_token_id") or [])))
    else:
        a.eos_ids = list(a.eos_id)
    if a.vocab_size is None:
        a.vocab_size = config_utils.get_vocab_size(a.model_dir) if cfg is None else cfg.get("vocab_size")
    if a.data_type is None:
        a.data_type = config_utils.get_dtype(a.model_dir) if cfg is None else cfg.get("torch_dtype", "bfloat16")
    # ---- scheduler defaults ----
    if a.router_token_ratio is None:
        a.router_token_ratio = 0.0 if a.run_mode in ("prefill", "decode") else 0.85
    if a.performance_mode == "personal":
        a.graph_max_batch_size = min(a.graph_max_batch_size, 16)
        a.running_max_req_size = min(a.running_max_req_size, 16)
        a.disable_chunked_prefill = True
    if a.batch_max_tokens is None:
        a.batch_max_tokens = max(16384 // a.dp, 1024) if not a.disable_chunked_prefill else \
            max(a.max_req_total_len, 16384 // a.dp)
    if a.chunked_prefill_size is None:
        a.chunked_prefill_size = a.batch_max_tokens if a.disable_chunked_prefill else max(a.batch_max_tokens // 2, 256)
    if not a.disable_chunked_prefill:
        assert a.batch_max_tokens >= a.chunked_prefill_size, "batch_max_tokens must cover chunked_prefill_size"
    else:
        assert a.batch_max_tokens >= a.max_req_total_len, "without chunked prefill batch_max_tokens must cover max_req_total_len"
    if a.graph_max_len_in_batch == 0:
        a.graph_max_len_in_batch = a.max_req_total_len
    # ---- mode compatibility ----
    if a.enable_prefill_microbatch_overlap or a.enable_decode_microbatch_overlap:
        a.enable_tpsp_mix_mode = True
    if a.use_dynamic_prompt_cache:
        a.disable_dynamic_prompt_cache = False
    if a.diverse_mode:
        assert not a.disable_dynamic_prompt_cache, "diverse_mode needs the prompt cache"
    if a.token_healing_mode:
        assert a.output_constraint_mode == "none", "token healing and output constraints are exclusive"
    assert not (a.first_token_constraint_mode and a.output_constraint_mode != "none")
    if a.enable_ep_moe:
        assert a.tp % a.dp == 0, "--enable_ep_moe: --dp must divide --tp (replicas of tp / dp tensor-parallel ranks)"
    if a.mtp_mode is not None:
        assert a.mtp_step > 0 and a.mtp_draft_model_dir, "mtp needs --mtp_step and --mtp_draft_model_dir"
    if a.run_mode in ("prefill", "decode"):
        via_config = bool(getattr(a, "config_server_host", None) and getattr(a, "config_server_port", None))
        assert via_config or (a.pd_master_ip and a.pd_master_port), \
            "PD nodes need --pd_master_ip / --pd_master_port, or --config_server_host / --config_server_port where the pd_masters register"
        # inherited by the model-rank processes (engine/pd/kv_transport.py:auth_key): what all nodes of the
        # deployment have in common
        os.environ["LLB_PD_MASTER_ADDR"] = f"{a.config_server_host}:{a.config_server_port}" if via_config else \
            f"{a.pd_master_ip}:{a.pd_master_port}"
        if getattr(a, "pd_kv_auth_key", None):
            os.environ["LLB_PD_KV_AUTHKEY"] = a.pd_kv_auth_key
        elif not os.environ.get("LLB_PD_KV_AUTHKEY"):
            print("[start] no --pd_kv_auth_key: the KV-transfer links are keyed by the pd_master (or config server) address only",
                  flush=True)
    # ---- names and ports ----
    if a.unique_server_name is None:
        a.unique_server_name = f"llb{os.getpid()}x{uuid.uuid4().hex[:6]}"
    os.environ["LIGHTLLM_UNIQUE_SERVICE_NAME_ID"] = a.unique_server_name
    need = ["router_port", "detokenization_port", "http_server_port", "metric_port", "visual_port", "audio_port",
            "cache_port", "multi_level_kv_cache_port"]
    missing = [n for n in need if getattr(a, n) is None]
    extra = 1 if a.nccl_port is None else 0
    ports = alloc_can_use_network_port(len(missing) + extra, used_ports=[a.port], start=20000 + (os.getpid() % 2000) * 10)
    for n, p in zip(missing, ports):
        setattr(a, n, p)
    if a.nccl_port is None:
        a.nccl_port = ports[-1]
    if a.run_mode == "decode":
        from ..utils.net_utils import alloc_consecutive_ports

        if a.pd_kv_port is None:  # rank r of this node receives KV pages on pd_kv_port + r
            a.pd_kv_port = alloc_consecutive_ports(a.tp, start=30000 + (os.getpid() % 2000) * 10, used_ports=ports)
        if a.pd_kv_status_port is None:
            a.pd_kv_status_port = alloc_can_use_network_port(1, used_ports=ports + [a.port], start=a.pd_kv_port + a.tp)[0]
    if a.disable_vision is None:
        a.disable_vision = True if cfg is not None else not config_utils.is_multimodal(a.model_dir)
    if a.disable_audio is None:
        a.disable_audio = True
    a.enable_multimodal = not a.disable_vision
    return a


def start_core_processes(args: StartArgs, config_override: dict = None):
    """Everything except the HTTP workers; returns when all of them reported "init ok"."""
    from .detokenization.manager import start_detokenization_process
    from .metrics.manager import start_metric_manager
    from .router.manager import start_router_process

    d = args.to_dict()
    d = {k: v for k, v in d.items() if not k.startswith("_")}
    # processes that do not depend on each other start (and import their libraries) side by side; the embedding
    # arena must exist before the ranks and the visual server open it, so with multimodal input there are two stages
    funcs, fargs = [start_metric_manager, start_detokenization_process], [(d,), (d,)]
    if args.enable_multimodal:
        from ..models.base import embed_row_width, load_config
        from .embed_cache.manager import start_cache_manager

        hidden = embed_row_width(config_override or load_config(args.model_dir))
        funcs.append(start_cache_manager)
        fargs.append((d, hidden))
        process_manager.start_submodule_processes(funcs, fargs)
        funcs, fargs = [], []
    funcs.append(start_router_process)
    fargs.append((d, config_override))
    if args.enable_multimodal:
        if getattr(args, "visual_use_proxy_mode", False):
            from .visualserver.remote import start_proxy_visual_process as start_visual_process
        else:
            from .visualserver.manager import start_visual_process

        dv = dict(d)
        dv["_config_override"] = config_override
        funcs.append(start_visual_process)
        fargs.append((dv,))
        if getattr(args, "enable_multimodal_audio", False):
            from .audioserver.manager import start_audio_process

            funcs.append(start_audio_process)
            fargs.append((dv,))
    process_manager.start_submodule_processes(funcs, fargs)


def run_http_server(args: StartArgs):
    import uvicorn

    set_env_start_args(args)
    from .httpserver.pd_loop import ws_max_size

    # websocket frames from prefill / decode nodes (prompt ids of long prompts): 128 MB unless the variable says otherwise
    uvicorn.run("lightllm_b200.server.api_http:app", host=args.host, port=args.port, workers=args.httpserver_workers,
                log_level="warning", loop="uvloop", timeout_keep_alive=5, ws_max_size=ws_max_size() or (128 << 20))


def normal_or_p_d_start(args: StartArgs, config_override: dict = None):
    set_proc_title(f"lightllm::{args.model_name}::api_server")
    require_free_ports(args.host, [args.port], "HTTP server")
    if config_override is None and args.model_dir and not os.path.isfile(os.path.join(args.model_dir, "config.json")):
        raise SystemExit(f"[lightllm_b200] --model_dir {args.model_dir}: no config.json there")
    args = normalize_args(args, config_override)
    set_env_start_args(args)
    from ..utils.shm_cleanup import check_shm_size, note_or_sweep_orphans

    if not getattr(args, "disable_shm_warning", False):
        check_shm_size(args)      # a warning when /dev/shm is smaller than the configuration wants
        note_or_sweep_orphans()   # segments of servers that were killed outright: said, or removed when asked to
    start_core_processes(args, config_override)
    if args.health_monitor:
        from .health_monitor.manager import start_health_check_process

        process_manager.start_submodule_processes([start_health_check_process], [(args.to_dict(),)])
    _watch_children()
    try:
        run_http_server(args)
    finally:
        process_manager.terminate_all()


def pd_master_start(args: StartArgs):
    require_free_ports(args.host, [args.port], "pd_master")
    args = normalize_args(args, {"vocab_size": None})
    set_env_start_args(args)
    from .metrics.manager import start_metric_manager

    process_manager.start_submodule_processes([start_metric_manager], [(args.to_dict(),)])
    _watch_children()
    try:
        run_http_server(args)
    finally:
        process_manager.terminate_all()


def _watch_children(interval_s: float = 1.0, grace_s: float = 15.0):
    """The HTTP server occupies the launcher's main thread, so a daemon thread watches the other processes: when
    one of them dies the server is no use any more (there is no in-process recovery of a lost rank), so the launcher
    stops the HTTP server, tears the remaining processes down and exits non-zero; whatever supervises the deployment
    restarts it.  Reference: lightllm/utils/start_utils.py:113-160."""
    import signal
    import threading

    def watch():
        while True:
            time.sleep(interval_s)
            dead = process_manager.any_dead()
            if dead is None:
                continue
            print(f"[launcher] a server process died ({dead}): shutting everything down", flush=True)
            process_manager.terminate_all()
            os.kill(os.getpid(), signal.SIGTERM)      # lets the HTTP server close its sockets and workers
            time.sleep(grace_s)
            os._exit(1)

    threading.Thread(target=watch, daemon=True, name="child-watch").start()


def config_server_start(args: StartArgs):
    import uvicorn

    from .config_server.api_http import app as cfg_app

    set_env_start_args(args)
    uvicorn.run(cfg_app, host=args.config_server_host or args.host, port=args.config_server_port or args.port,
                log_level="warning")


def visual_only_start(args: StartArgs, config_override: dict = None):
    """A vision encoder on its own: it registers at the config server and embeds pictures for the servers that run
    with `--visual_use_proxy_mode` (reference: api_start.py visual_only_start)."""
    from .visualserver.remote import start_visual_only_process

    args = normalize_args(args, config_override)
    if getattr(args, "afs_image_embed_dir", None):
        os.makedirs(args.afs_image_embed_dir, mode=0o777, exist_ok=True)
    set_env_start_args(args)
    d = {k: v for k, v in args.to_dict().items() if not k.startswith("_")}
    d["_config_override"] = config_override
    process_manager.start_submodule_processes([start_visual_only_process], [(d,)])
    process_manager.supervise()
