"""Reference arm of bench.py: the unmodified reference engine on the same workload.

The reference package is installed under ``baseline/_ref`` (pip, --no-deps, from a copy of the
read-only source tree).  Its third-party pure-Python dependencies that are absent from the offline
image (easydict, frozendict, orjson, ujson, rpyc, atomics, librosa, soxr, cupy) are satisfied by small
stand-ins in ``baseline/shims``; none of this repository's models, kernels or engine is on the path.

The run goes through the reference's own engine API, the way its static benchmark does
(test/benchmark/static_inference/static_benchmark.py): launch arguments from its argparse,
``set_env_start_args``, ``init_distributed_env``, ``get_model`` -> ``TpPartBaseModel`` with its
stock kernels (cuBLAS GEMM, FlashInfer / Triton attention, Triton elementwise ops, its all-reduce
dispatch, decode CUDA graphs), ``model.forward(ModelInput)``.  Workload and timing are those of the
other arm: one step = one wave of `conc` requests (prefill passes of batch_max_tokens tokens, then
out_len - 1 decode steps at batch `conc`), greedy sampling on the device, CUDA events, max over
ranks.  Weights are random (N(0, 0.02), same shapes) handed to the model as its `weight_dict`.
"""
from __future__ import annotations

import json
import os
import sys
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))


def _unavailable(why: str):
    print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:400]}), flush=True)


def _random_weight_dict(cfg: dict, device, dtype):
    import torch

    H, L = cfg["hidden_size"], cfg["num_hidden_layers"]
    D = cfg.get("head_dim") or H // cfg["num_attention_heads"]
    nq, nkv, I, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"], cfg["vocab_size"]
    g = torch.Generator(device=device)
    g.manual_seed(0)

    def w(*shape):
        return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * 0.02).to(dtype)

    d = {"model.embed_tokens.weight": w(V, H), "model.norm.weight": torch.ones(H, dtype=dtype, device=device),
         "lm_head.weight": w(V, H)}
    for i in range(L):
        p = f"model.layers.{i}."
        d[p + "input_layernorm.weight"] = torch.ones(H, dtype=dtype, device=device)
        d[p + "post_attention_layernorm.weight"] = torch.ones(H, dtype=dtype, device=device)
        d[p + "self_attn.q_proj.weight"] = w(nq * D, H)
        d[p + "self_attn.k_proj.weight"] = w(nkv * D, H)
        d[p + "self_attn.v_proj.weight"] = w(nkv * D, H)
        d[p + "self_attn.o_proj.weight"] = w(H, nq * D)
        d[p + "mlp.gate_proj.weight"] = w(I, H)
        d[p + "mlp.up_proj.weight"] = w(I, H)
        d[p + "mlp.down_proj.weight"] = w(H, I)
    return d


def _run(args, MODELS):
    sys.path.insert(0, os.path.join(HERE, "shims"))
    sys.path.insert(0, os.path.join(HERE, "_ref"))
    import numpy as np
    import torch

    if not torch.cuda.is_available():
        return _unavailable("no CUDA device")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    assert world == args.gpus
    cfg = dict(MODELS[args.model])
    cfg.setdefault("architectures", ["LlamaForCausalLM"])
    cfg.setdefault("max_position_embeddings", 8192)
    conc, in_len, out_len = args.conc, args.in_len, args.out_len
    total_len = in_len + out_len
    model_dir = f"/tmp/llb_ref_model_{os.getpid()}"
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f)

    os.environ.setdefault("LIGHTLLM_LOG_LEVEL", "warning")
    os.environ["DISABLE_CHECK_MAX_LEN_INFER"] = "1"
    from lightllm.server.api_cli import make_argument_parser
    from lightllm.utils.envs_utils import set_env_start_args

    # Under torch.distributed.run the workers inherit TORCHELASTIC_USE_AGENT_STORE=True, which makes torch's
    # tcp:// rendezvous (the reference's init_process_group in lightllm/utils/dist_utils.py:150-155) connect EVERY
    # rank as a client of nccl_host:nccl_port and start no server there, so all ranks wait for a store nobody
    # serves.  The reference is normally started by its own launcher, without an elastic agent: drop the variable
    # so that rank 0 hosts the store on the port it is given.
    os.environ.pop("TORCHELASTIC_USE_AGENT_STORE", None)
    port = int(os.environ.get("MASTER_PORT", "29500")) + 37
    ref_args = make_argument_parser().parse_args([
        "--model_dir", model_dir, "--tp", str(world), "--data_type", "bf16",
        "--max_total_token_num", str(conc * (total_len + 8) + args.batch_max_tokens),
        "--running_max_req_size", str(conc), "--batch_max_tokens", str(args.batch_max_tokens),
        "--max_req_total_len", str(total_len + 8), "--graph_max_batch_size", str(conc),
        "--nccl_host", os.environ.get("MASTER_ADDR", "127.0.0.1"), "--nccl_port", str(port)])
    ref_args.graph_max_len_in_batch = total_len + 8
    ref_args.chunked_prefill_size = args.batch_max_tokens // 2
    ref_args.router_token_ratio = 0.85
    ref_args.eos_id = [cfg["eos_token_id"]]
    ref_args.enable_multimodal = False
    ref_args.enable_multimodal_audio = False
    from easydict import EasyDict

    set_env_start_args(EasyDict(vars(ref_args)))

    from lightllm.common.basemodel.batch_objs import ModelInput
    from lightllm.distributed import dist_group_manager
    from lightllm.models import get_model
    from lightllm.utils.dist_utils import init_distributed_env

    kvargs = {
        "args": ref_args, "nccl_host": ref_args.nccl_host, "nccl_port": ref_args.nccl_port, "rank_id": rank,
        "world_size": world, "dp_size": 1, "weight_dir": model_dir, "data_type": "bf16", "quant_type": "none",
        "quant_cfg": None, "expert_dtype": None, "load_way": "HF",
        "max_total_token_num": ref_args.max_total_token_num, "graph_max_len_in_batch": total_len + 8,
        "graph_max_batch_size": conc, "mem_fraction": 0.9, "max_req_num": conc,
        "batch_max_tokens": args.batch_max_tokens, "run_mode": "normal", "max_seq_length": total_len + 8,
        "disable_cudagraph": False, "llm_prefill_att_backend": ref_args.llm_prefill_att_backend,
        "llm_decode_att_backend": ref_args.llm_decode_att_backend, "vit_att_backend": ref_args.vit_att_backend,
        "llm_kv_type": ref_args.llm_kv_type, "llm_kv_quant_group_size": ref_args.llm_kv_quant_group_size,
    }
    init_distributed_env(kvargs)
    dist_group_manager.create_groups(group_size=1)
    dev = torch.device("cuda", torch.cuda.current_device())
    kvargs["weight_dict"] = _random_weight_dict(cfg, dev, torch.bfloat16)
    model, _ = get_model(cfg, kvargs)
    kvargs["weight_dict"] = None
    torch.cuda.empty_cache()

    rm, mm = model.req_manager, model.req_manager.mem_manager
    req_idx = torch.tensor([rm.alloc() for _ in range(conc)], dtype=torch.int32)
    per_pass = max(1, args.batch_max_tokens // in_len)
    rng = np.random.default_rng(1234)

    def i32(n, v):
        return torch.full((n,), v, dtype=torch.int32).pin_memory()

    # Inputs of a wave that do not depend on the prompts, staged once in pinned host memory (the other arm does
    # the same): request rows, lengths, start offsets.  The reference's ModelInput.to_cuda() copies them with
    # .cuda(non_blocking=True) inside forward.
    no_mm_prefill = {}
    pre = []
    for s0 in range(0, conc, per_pass):
        e0 = min(conc, s0 + per_pass)
        B = e0 - s0
        b_seq = i32(B, in_len)
        pre.append((s0, e0, B, b_seq, i32(B, 0), (torch.arange(B, dtype=torch.int32) * in_len).pin_memory(),
                    req_idx[s0:e0].clone().pin_memory(), i32(B, 0)))
        no_mm_prefill[B] = [{"images": [], "audios": []} for _ in range(B)]
    no_mm_decode = [{"images": [], "audios": []} for _ in range(conc)]
    dec_req = req_idx.clone().pin_memory()
    dec_zero = i32(conc, 0)
    dec_seq = [i32(conc, in_len + t) for t in range(out_len)]
    ring = [torch.empty(conc, dtype=torch.int64).pin_memory() for _ in range(4)]
    io = {"h2d": 0, "d2h": 0, "passes": 0}

    def nbytes(*ts):
        return sum(t.numel() * t.element_size() for t in ts)

    def wave(prompts_np, e2e=False):
        """One wave.  e2e=False: sampled ids stay on the device between steps (device-timed `value`, same
        treatment as the other arm's loop).  e2e=True: additionally every step's sampled ids are copied to pinned
        host memory and read there before the step after next is issued (what a serving loop needs for stop
        checks and streaming), and the copies are counted."""
        mm.free_all()
        slots = mm.alloc(conc * total_len).view(conc, total_len)
        slots_t = slots.t().contiguous().pin_memory()          # [position, request]
        prompts = torch.from_numpy(prompts_np).pin_memory()
        next_ids = torch.empty(conc, dtype=torch.int64, device=dev)
        pending = []
        for s0, e0, B, b_seq, b_ready, start_loc, reqs_p, mtp0 in pre:
            mem = slots[s0:e0, :in_len].reshape(-1).contiguous().pin_memory()
            ids = prompts[s0:e0].reshape(-1)
            mi = ModelInput(batch_size=B, total_token_num=B * in_len, max_q_seq_len=in_len, max_kv_seq_len=in_len,
                            max_cache_len=0, prefix_total_token_num=0, input_ids=ids, b_req_idx=reqs_p,
                            b_mtp_index=mtp0, b_seq_len=b_seq, mem_indexes_cpu=mem, is_prefill=True,
                            b_ready_cache_len=b_ready, b_prefill_start_loc=start_loc,
                            b_prefill_has_output_cpu=[True] * B, multimodal_params=no_mm_prefill[B])
            if e2e:
                io["h2d"] += nbytes(ids, reqs_p, mtp0, b_seq, mem, b_ready, start_loc)
                io["passes"] += 1
            out = model.forward(mi)
            next_ids[s0:e0] = torch.argmax(out.logits, dim=-1)
        for t in range(1, out_len):
            L = in_len + t
            mem = slots_t[L - 1]
            mi = ModelInput(batch_size=conc, total_token_num=conc * L, max_q_seq_len=1, max_kv_seq_len=L,
                            input_ids=next_ids, b_req_idx=dec_req, b_mtp_index=dec_zero, b_seq_len=dec_seq[t],
                            b_position_delta=dec_zero, mem_indexes_cpu=mem, is_prefill=False,
                            multimodal_params=no_mm_decode)
            out = model.forward(mi)
            next_ids = torch.argmax(out.logits, dim=-1)
            if e2e:
                io["h2d"] += nbytes(dec_req, dec_zero, dec_seq[t], dec_zero, mem)
                io["d2h"] += conc * 8
                io["passes"] += 1
                host = ring[t % 4]
                host.copy_(next_ids, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
                pending.append((ev, host))
                if len(pending) > 1:       # the previous step's ids are read while this step runs
                    pev, ph = pending.pop(0)
                    pev.synchronize()
                    int(ph[0])
        for pev, ph in pending:
            pev.synchronize()
            int(ph[0])
        return next_ids

    def new_prompts():
        return rng.integers(1000, cfg["vocab_size"] - 1000, size=(conc, in_len), dtype=np.int64)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        wave(new_prompts())
    barrier()
    from bench import ClockSampler, bench_config

    clocks = ClockSampler(dev.index or 0)
    clocks.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        wave(new_prompts())
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clock_info = clocks.stop()
    wall = 0.0
    if not args.skip_e2e:
        wave(new_prompts(), e2e=True)
        io.update(h2d=0, d2h=0, passes=0)
        barrier()
        t0 = time.time()
        for _ in range(args.steps):
            wave(new_prompts(), e2e=True)
        barrier()
        wall = time.time() - t0
    v = torch.tensor([ms, wall], dtype=torch.float64, device=dev)
    if world > 1:
        torch.distributed.all_reduce(v, op=torch.distributed.ReduceOp.MAX)
    ms, wall = float(v[0]), float(v[1])
    out_tokens = args.steps * conc * out_len
    if rank == 0:
        line = {
            "metric": "output tok/s per box at fixed concurrency", "value": round(out_tokens / (ms / 1e3), 1),
            "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms / args.steps, 2), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
            "impl": "reference", "config": bench_config(args),
            "engine": {"prefill_att_backend": type(model.prefill_att_backend).__name__,
                       "decode_att_backend": type(model.decode_att_backend).__name__},
            "clocks": clock_info,
        }
        if wall > 0:
            line["e2e"] = {"value": round(out_tokens / wall, 1), "unit": "tokens/s",
                           "h2d_bytes_per_step": round(io["h2d"] / max(io["passes"], 1), 1),
                           "d2h_bytes_per_step": round(io["d2h"] / max(io["passes"], 1), 1),
                           "bytes_are_per": "forward pass (prefill chunk or decode step)",
                           "note": "the reference's engine API driven like a serving loop on the host clock (its HTTP "
                                   "server needs rpyc / hypercorn, absent offline): every pass copies its inputs from "
                                   "pinned host memory (ModelInput.to_cuda) and every decode step's sampled ids go "
                                   "back to pinned host memory and are read there one step later"}
        print(json.dumps(line), flush=True)


def main(args, MODELS):
    if not os.path.isdir(os.path.join(HERE, "_ref", "lightllm")):
        return _unavailable("baseline/_ref is missing: pip install --no-index --no-deps --target baseline/_ref of the "
                            "reference was not done in this checkout")
    try:
        _run(args, MODELS)
    except BaseException as e:  # the reference may raise anything, including SystemExit from its own watchdogs
        tb = traceback.format_exc()
        sys.stderr.write(tb)
        _unavailable(f"reference engine failed on this box: {type(e).__name__}: {e}")
