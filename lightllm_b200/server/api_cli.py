"""Launch flags of ``python -m lightllm_b200.server.api_server``.

The flag surface (names, types, defaults, choices) is the one users of the reference already
have in their launch scripts (lightllm/server/api_cli.py); flags that select between kernel
back-ends are accepted for compatibility and documented as having a single implementation
here (this package has one sm_100a code path per op).

Flags are declared in one table: (name, kind, default, help[, extra]) with kind one of
int / float / str / "flag" (store_true) / ("list", type) (nargs="+") / "append".
"""
from __future__ import annotations

import argparse

TOOL_PARSERS = ["qwen25", "llama3", "mistral", "deepseekv3", "qwen", "deepseekv31", "deepseekv32", "glm47", "kimi_k2",
                "qwen3_coder"]
REASONING_PARSERS = ["deepseek-r1", "deepseek-v3", "glm45", "gpt-oss", "kimi", "kimi_k2", "qwen3", "qwen3-thinking",
                     "minimax", "minimax-append-think", "step3", "nano_v3", "interns1", "gemma4"]

FLAGS = [
    # ---- mode ----
    ("--run_mode", str, "normal", "normal serving, or the roles of prefill/decode disaggregation "
     "(prefill, decode, pd_master), the config_server registry, or a stand-alone visual encoder (visual_only)",
     dict(choices=["normal", "prefill", "decode", "pd_master", "config_server", "visual_only"])),
    ("--performance_mode", str, None, "'personal': latency-oriented preset for a single user "
     "(small graphs, no chunk splitting)", dict(choices=["personal"])),
    # ---- network ----
    ("--host", str, "127.0.0.1", "HTTP bind address"),
    ("--port", int, 8000, "HTTP port"),
    ("--httpserver_workers", int, 1, "number of HTTP worker processes"),
    ("--hypercorn_config", str, None, "TOML file with extra HTTP server settings (keep-alive, backlog, ...)"),
    ("--zmq_mode", str, "ipc:///tmp/", "zmq transport prefix between the processes of a node: ipc:///tmp/ or tcp://"),
    ("--nccl_host", str, "127.0.0.1", "rendezvous address of the model ranks"),
    ("--nccl_port", int, None, "rendezvous port of the model ranks (picked automatically when unset)"),
    ("--use_config_server_to_init_nccl", "flag", False, "take the rendezvous store from the config server"),
    ("--nnodes", int, 1, "number of nodes of a multi-node tensor-parallel deployment"),
    ("--node_rank", int, 0, "rank of this node"),
    ("--multinode_httpmanager_port", int, 12345, "node 0 forwards raw requests to the other nodes on this port"),
    ("--multinode_router_gloo_port", int, 20001, "port of the gloo group that keeps the routers of all nodes identical"),
    # ---- PD disaggregation ----
    ("--pd_master_ip", str, "0.0.0.0", "address of the pd_master (prefill/decode nodes register there)"),
    ("--pd_master_port", int, 1212, "port of the pd_master"),
    ("--pd_master_mode", str, "elastic", "'elastic' (nodes may join and leave) or a fixed topology such as 2p4d"),
    ("--pd_trans_mode", str, "nccl", "KV transfer transport between prefill and decode nodes",
     dict(choices=["nccl", "nixl"])),
    ("--select_p_d_node_strategy", str, "cache_aware", "how the pd_master picks a (prefill, decode) pair",
     dict(choices=["random", "round_robin", "adaptive_load", "cache_aware"])),
    ("--config_server_host", str, None, "config server address (several pd_masters / remote ViT)"),
    ("--config_server_port", int, None, "config server port"),
    ("--config_server_visual_redis_port", int, None, "redis port used by remote visual encoders"),
    ("--pd_kv_page_num", int, 16, "staging pages of the KV mover"),
    ("--pd_kv_page_size", int, 1024, "tokens per staging page"),
    ("--pd_kv_auth_key", str, None, "shared secret of the KV-transfer control connections; give every prefill and "
     "decode node of one deployment the same value (or set LLB_PD_KV_AUTHKEY)"),
    # ---- model ----
    ("--model_name", str, "default_model_name", "name reported by /v1/models"),
    ("--model_owner", str, None, "owner reported by /v1/models"),
    ("--model_dir", str, None, "HuggingFace model directory (config.json, tokenizer, *.safetensors)"),
    ("--tokenizer_mode", str, "fast", "fast | slow | auto"),
    ("--load_way", str, "HF", "checkpoint format (HF)"),
    ("--trust_remote_code", "flag", False, "allow custom tokenizer / config code from the model directory"),
    ("--data_type", str, None, "activation dtype (defaults to the checkpoint's)",
     dict(choices=["fp16", "float16", "bf16", "bfloat16", "fp32", "float32"])),
    ("--eos_id", ("list", int), None, "end-of-sequence token id(s); default from config.json"),
    ("--chat_template", str, None, "jinja chat template file overriding the tokenizer's"),
    ("--tool_call_parser", str, None, "tool-call syntax of the model for /v1/chat/completions",
     dict(choices=TOOL_PARSERS)),
    ("--reasoning_parser", str, None, "reasoning-content syntax of the model", dict(choices=REASONING_PARSERS)),
    # ---- capacity ----
    ("--max_total_token_num", int, None, "size of the KV pool in tokens; default: profiled from free memory"),
    ("--mem_fraction", float, 0.8, "fraction of free device memory given to the KV pool when profiling"),
    ("--max_req_total_len", int, None, "longest prompt + output of one request; default from the model config"),
    ("--running_max_req_size", int, 256, "maximum number of requests in flight (also the number of shm request slots)"),
    ("--batch_max_tokens", int, None, "token budget of one prefill pass; default 16384 / dp"),
    ("--chunked_prefill_size", int, None, "largest prompt chunk of one request per pass; default batch_max_tokens/2"),
    ("--disable_chunked_prefill", "flag", False, "prefill every prompt in a single pass"),
    # ---- parallelism ----
    ("--tp", int, 1, "total number of GPUs (world size)"),
    ("--dp", int, 1, "data-parallel attention replicas; each replica is a tensor-parallel group of tp/dp ranks"),
    ("--dp_balancer", str, "bs_balancer", "request placement across replicas",
     dict(choices=["round_robin", "bs_balancer"])),
    ("--enable_tpsp_mix_mode", "flag", False, "token-sharded residual stream: reduce-scatter after o_proj/down_proj, "
     "all-gather before qkv/gate_up"),
    ("--enable_dp_prefill_balance", "flag", False, "re-balance prefill tokens across replicas"),
    ("--enable_ep_moe", "flag", False, "expert parallelism for MoE layers (use with --dp equal to --tp)"),
    ("--enable_prefill_microbatch_overlap", "flag", False, "two prefill micro-batches overlap compute and communication"),
    ("--enable_decode_microbatch_overlap", "flag", False, "two decode micro-batches overlap compute and communication"),
    ("--ep_redundancy_expert_config_path", str, None, "JSON with redundant expert placement"),
    ("--auto_update_redundancy_expert", "flag", False, "re-place redundant experts from live usage counters"),
    ("--enable_fused_shared_experts", "flag", False, "treat the shared expert as one more routed expert (TP MoE)"),
    ("--expert_dtype", str, None, "quantise expert weights at load", dict(choices=["fp8", "fp4"])),
    # ---- scheduler ----
    ("--router_token_ratio", float, None, "pool usage above which the router assumes every request runs to its "
     "max_new_tokens; default 0.85 (0.0 on prefill/decode nodes)"),
    ("--router_max_wait_tokens", int, 1, "decode steps between two prefill passes when not scheduling aggressively"),
    ("--disable_aggressive_schedule", "flag", False, "do not prefill as soon as a request is admitted"),
    ("--enable_prefill_decode_mixed", "flag", False, "allow prefill chunks and decode rows in one pass"),
    ("--schedule_time_interval", float, 0.03, "router period in seconds"),
    ("--use_dynamic_prompt_cache", "flag", False, "kept for compatibility (prefix caching is on by default)"),
    ("--disable_dynamic_prompt_cache", "flag", False, "turn the radix prefix cache off"),
    ("--diverse_mode", "flag", False, "n>1 samples share the prompt's KV"),
    ("--token_healing_mode", "flag", False, "regenerate the last prompt tokens under a prefix constraint"),
    ("--output_constraint_mode", str, "none", "constrained decoding engine",
     dict(choices=["outlines", "xgrammar", "none"])),
    ("--first_token_constraint_mode", "flag", False, "restrict the first generated token (env FIRST_ALLOWED_TOKENS)"),
    # ---- kernels ----
    ("--llm_prefill_att_backend", ("list", str), ["auto"], "accepted for compatibility: prefill attention is this "
     "package's paged sm_100a kernel", dict(choices=["auto", "triton", "fa3", "flashinfer", "flashqla"])),
    ("--llm_decode_att_backend", ("list", str), ["auto"], "accepted for compatibility: decode attention is this "
     "package's paged split-KV kernel", dict(choices=["auto", "triton", "fa3", "flashinfer"])),
    ("--vit_att_backend", ("list", str), ["auto"], "attention of the visual encoder",
     dict(choices=["auto", "triton", "fa3", "sdpa", "xformers"])),
    ("--llm_kv_type", str, "None", "KV cache storage type",
     dict(choices=["None", "int8kv", "int4kv", "fp8kv_sph", "fp8kv_spt", "fp8kv_dsa"])),
    ("--llm_kv_quant_group_size", int, 8, "group size of int8/int4 KV quantisation"),
    ("--kv_quant_calibration_config_path", str, None, "JSON with calibrated fp8 KV scales"),
    ("--quant_type", str, "none", "weight quantisation: none | fp8w8a8-b128 (e4m3, 128x128 block scales) | ..."),
    ("--quant_cfg", str, None, "YAML with per-layer quantisation overrides"),
    ("--vit_quant_type", str, "none", "quantisation of the visual encoder"),
    ("--vit_quant_cfg", str, None, "YAML with per-layer overrides for the visual encoder"),
    ("--sampling_backend", str, "triton", "accepted for compatibility: sampling is this package's fused kernel",
     dict(choices=["triton", "flashinfer"])),
    ("--penalty_counter_mode", str, "gpu_counter", "where per-request token counters for penalties live",
     dict(choices=["cpu_counter", "pin_mem_counter", "gpu_counter"])),
    ("--disable_symm_mem_allreduce", "flag", False, "do not use the peer-memory (NVLink) fused all-reduce kernels"),
    ("--disable_flashinfer_allreduce", "flag", False, "accepted for compatibility (one-shot all-reduce is in-tree)"),
    ("--hardware_platform", str, "cuda", "cuda", dict(choices=["cuda", "musa"])),
    ("--enable_torch_fallback", "flag", False, "run ops through their plain PyTorch restatements (debugging)"),
    ("--enable_triton_fallback", "flag", False, "accepted for compatibility (no Triton in this package)"),
    # ---- CUDA graphs ----
    ("--disable_cudagraph", "flag", False, "launch decode eagerly instead of replaying CUDA graphs"),
    ("--graph_max_batch_size", int, 256, "largest decode batch captured as a graph"),
    ("--graph_split_batch_size", int, 32, "every batch size up to this one gets its own graph"),
    ("--graph_grow_step_size", int, 16, "bucket step above graph_split_batch_size"),
    ("--graph_max_len_in_batch", int, 0, "longest sequence a graph may serve; 0 = max_req_total_len"),
    ("--enable_prefill_cudagraph", "flag", False, "piecewise CUDA graphs for prefill"),
    ("--prefill_cudagraph_max_handle_token", int, 8192, "largest prefill pass served by a graph"),
    # ---- speculative decoding ----
    ("--mtp_mode", str, None, "multi-token prediction mode",
     dict(choices=["vanilla_with_att", "eagle_with_att", "vanilla_no_att", "eagle_no_att", None])),
    ("--mtp_draft_model_dir", ("list", str), None, "draft model directory(ies)"),
    ("--mtp_step", int, 0, "draft tokens per step"),
    # ---- caches ----
    ("--enable_cpu_cache", "flag", False, "second-level KV cache in pinned host memory"),
    ("--cpu_cache_storage_size", float, 2, "host KV cache size in GB"),
    ("--cpu_cache_token_page_size", int, 256, "tokens per host cache page"),
    ("--enable_disk_cache", "flag", False, "third-level KV cache on disk"),
    ("--disk_cache_storage_size", float, 10, "disk KV cache size in GB"),
    ("--disk_cache_dir", str, None, "directory of the disk KV cache"),
    ("--enable_dp_prompt_cache_fetch", "flag", False, "fetch cached prefixes from other replicas over peer memory"),
    ("--linear_att_hash_page_size", int, 512, "page size of the linear-attention state cache"),
    ("--linear_att_page_block_num", int, 10000000, "pages of the linear-attention state cache"),
    ("--linear_att_cache_size", int, None, "state slots of hybrid linear-attention models"),
    ("--linear_att_ssm_data_type", str, "float32", "dtype of the recurrent state", dict(choices=["bfloat16", "float32"])),
    ("--disable_linear_att_small_page_cpu_cache", "flag", False, "do not offload small state pages"),
    # ---- multimodal ----
    ("--disable_vision", "flag", None, "do not start the visual encoder"),
    ("--disable_audio", "flag", None, "do not start the audio encoder"),
    ("--enable_multimodal_url_cache", "flag", False, "cache downloaded images/audio by URL"),
    ("--enable_mps", "flag", False, "share GPUs between encoders and LLM ranks with MPS"),
    ("--cache_capacity", int, 200, "entries of the multimodal embedding cache"),
    ("--embed_cache_storage_size", float, 4, "embedding cache size in GB"),
    ("--max_image_token_count", int, 8192, "largest number of tokens one image may expand to"),
    ("--max_image_pixels", int, 3686400, "images above this pixel count are resized"),
    ("--disable_image_resize", "flag", False, "never resize images"),
    ("--visual_infer_batch_size", int, None, "images per encoder pass"),
    ("--visual_send_batch_size", int, 1, "requests forwarded to the router per message"),
    ("--visual_gpu_ids", ("list", int), None, "GPUs of the visual encoder"),
    ("--visual_tp", int, 1, "tensor parallel size of the visual encoder"),
    ("--visual_dp", int, 1, "replicas of the visual encoder"),
    ("--visual_rpyc_port", int, None, "--run_mode visual_only: the port this vision encoder is asked on"),
    ("--visual_use_proxy_mode", "flag", False, "keep no vision tower: pictures go to the encoders (--run_mode "
     "visual_only) registered at the config server"),
    ("--audio_gpu_ids", ("list", int), None, "GPUs of the audio encoder"),
    ("--audio_tp", int, 1, "tensor parallel size of the audio encoder"),
    ("--audio_dp", int, 1, "replicas of the audio encoder"),
    ("--audio_infer_batch_size", int, None, "clips per encoder pass"),
    ("--afs_image_embed_dir", str, None, "directory all servers see: image embeddings by content hash, shared "
     "between vision encoders and the servers that use them"),
    ("--afs_embed_capacity", int, 250000, "files kept in --afs_image_embed_dir (least recently used go first)"),
    # ---- operations ----
    ("--health_monitor", "flag", False, "watch /health and restart the server after repeated failures"),
    ("--metric_gateway", str, None, "Prometheus push gateway address"),
    ("--job_name", str, "lightllm", "job label for the push gateway"),
    ("--grouping_key", "append", [], "key=value grouping label (repeatable)"),
    ("--push_interval", int, 10, "push period in seconds"),
    ("--enable_monitor_auth", "flag", False, "authenticate against the push gateway"),
    ("--detail_log", "flag", False, "log per-request stage timings"),
    ("--disable_shm_warning", "flag", False, "do not warn about a small /dev/shm"),
    ("--enable_profiling", str, None, "expose /profiler_start and /profiler_stop",
     dict(choices=["torch_profiler", "nvtx"])),
    ("--use_reward_model", "flag", False, "serve a reward model (/get_score)"),
    ("--use_tgi_api", "flag", False, "TGI-compatible request/response format on /"),
    ("--enable_prompt_logprobs", "flag", False, "allow requests to ask for prompt logprobs"),
    ("--enable_return_routed_experts", "flag", False, "allow requests to ask for the routed expert ids"),
    # ---- RL ----
    ("--enable_rl", "flag", False, "weight-update / pause / flush control plane for RL trainers"),
    ("--enable_torch_memory_saver", "flag", False, "release and resume GPU memory on request"),
    ("--enable_weight_cpu_backup", "flag", False, "release_memory_occupation of the weights keeps a pinned host "
     "copy that resume restores (without it, resume hands out zeroed weights for the next push)"),
]


ALIASES = {"--performance_mode": ["--p_mode"]}     # short spellings the reference accepts


def add_cli_args(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    for spec in FLAGS:
        name, kind, default, help_ = spec[:4]
        extra = dict(spec[4]) if len(spec) > 4 else {}
        names = [name] + ALIASES.get(name, [])
        if kind == "flag":
            parser.add_argument(*names, action="store_true", default=default, help=help_)
        elif kind == "append":
            parser.add_argument(*names, action="append", default=default, help=help_)
        elif isinstance(kind, tuple):
            parser.add_argument(*names, type=kind[1], nargs="+", default=default, help=help_, **extra)
        else:
            parser.add_argument(*names, type=kind, default=default, help=help_, **extra)
    return parser


def make_argument_parser() -> argparse.ArgumentParser:
    return add_cli_args(argparse.ArgumentParser(prog="lightllm_b200.server.api_server",
                                                formatter_class=argparse.RawTextHelpFormatter))


# Accepted so that the reference's start scripts keep working; nothing in this package reads them.
COMPAT_ONLY_FLAGS = (
    "llm_prefill_att_backend", "llm_decode_att_backend", "vit_att_backend", "sampling_backend", "enable_torch_fallback",
    "enable_triton_fallback", "disable_flashinfer_allreduce", "penalty_counter_mode", "load_way",
    "enable_prefill_cudagraph", "prefill_cudagraph_max_handle_token",
    "pd_trans_mode",
    "config_server_visual_redis_port", "vit_quant_type", "vit_quant_cfg", "visual_tp", "audio_tp",
    "linear_att_page_block_num", "hypercorn_config", "enable_mps",
    "enable_torch_memory_saver")


def compat_only_flags_in_use(args) -> list:
    """Names of compatibility-only flags whose value differs from the default (for a start-up notice)."""
    defaults = {}
    for spec in FLAGS:
        name, kind, default = spec[0].lstrip("-"), spec[1], spec[2]
        defaults[name] = False if kind == "flag" else default
    used = []
    for name in COMPAT_ONLY_FLAGS:
        if name in defaults and getattr(args, name, defaults[name]) != defaults[name]:
            used.append(name)
    return used

