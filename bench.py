"""Serving benchmark: output tokens/s per box at fixed concurrency (plus p50 TTFT / ITL).

    python bench.py --gpus 1 --steps 2 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Workload (the Llama-3-8B serving configuration): Llama-3-8B architecture, bf16, random-init
weights, uniform-random token ids, fixed input 1024 / output 256 tokens, greedy, `--conc`
(256) requests in flight, tensor parallel over the N GPUs.  One *step* is one wave: `conc`
requests taken from arrival to their last token (16 chunked-prefill passes of 16384 tokens and
255 decode passes at batch 256, CUDA-graph replayed, sampling included); 2 steps are the 512
requests of the configuration.

Two measurements of the same metric:
  value : device-timed (CUDA events around K waves, max over ranks).  The wave is driven through
          the model runner with the sampled tokens staying on the device, so it is the kernel
          throughput of the whole serving step with no host round trip per token.
  e2e   : K waves through the public offline API `LLM.generate` (admission queue, radix cache,
          per-step H2D of the step's indices / prompt ids from pinned memory, per-step D2H of
          the sampled tokens, stop checks), host clock, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODELS = {
    "llama3-8b": dict(model_type="llama", hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
                      num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=128256,
                      rms_norm_eps=1e-5, rope_theta=5e5, eos_token_id=128001, torch_dtype="bfloat16"),
    "llama3-70b": dict(model_type="llama", hidden_size=8192, num_hidden_layers=80, num_attention_heads=64,
                       num_key_value_heads=8, head_dim=128, intermediate_size=28672, vocab_size=128256,
                       rms_norm_eps=1e-5, rope_theta=5e5, eos_token_id=128001, torch_dtype="bfloat16"),
    # Qwen3-30B-A3B shapes (128 routed experts, top-8 softmax routing with normalised weights)
    "qwen3-30b-a3b": dict(model_type="qwen3_moe", hidden_size=2048, num_hidden_layers=48, num_attention_heads=32,
                          num_key_value_heads=4, head_dim=128, intermediate_size=6144, moe_intermediate_size=768,
                          num_experts=128, num_experts_per_tok=8, norm_topk_prob=True, decoder_sparse_step=1,
                          mlp_only_layers=[], vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1e6, eos_token_id=151645,
                          torch_dtype="bfloat16"),
    # DeepSeek-V3 shapes, e4m3 weights with 128 x 128 block scales
    "deepseek-v3": dict(model_type="deepseek_v3", hidden_size=7168, num_hidden_layers=61, num_attention_heads=128,
                        num_key_value_heads=128, q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128,
                        qk_rope_head_dim=64, v_head_dim=128, intermediate_size=18432, moe_intermediate_size=2048,
                        n_routed_experts=256, n_shared_experts=1, num_experts_per_tok=8, n_group=8, topk_group=4,
                        first_k_dense_replace=3, moe_layer_freq=1, routed_scaling_factor=2.5, norm_topk_prob=True,
                        scoring_func="sigmoid", topk_method="noaux_tc", vocab_size=129280, rms_norm_eps=1e-6,
                        rope_theta=10000.0, eos_token_id=1, torch_dtype="bfloat16",
                        quantization_config={"quant_method": "fp8", "fmt": "e4m3", "activation_scheme": "dynamic",
                                             "weight_block_size": [128, 128]}),
    "tiny-moe": dict(model_type="qwen3_moe", hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=64, intermediate_size=512, moe_intermediate_size=128,
                     num_experts=8, num_experts_per_tok=2, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[],
                     vocab_size=1024, rms_norm_eps=1e-6, rope_theta=1e4, eos_token_id=2, torch_dtype="bfloat16"),
    "tiny-ds": dict(model_type="deepseek_v3", hidden_size=256, intermediate_size=512, moe_intermediate_size=128,
                    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, n_routed_experts=8,
                    n_shared_experts=1, num_experts_per_tok=2, n_group=2, topk_group=1, first_k_dense_replace=1,
                    q_lora_rank=128, kv_lora_rank=128, qk_nope_head_dim=64, qk_rope_head_dim=32, v_head_dim=64,
                    vocab_size=1024, routed_scaling_factor=2.5, norm_topk_prob=True, scoring_func="sigmoid",
                    topk_method="noaux_tc", rms_norm_eps=1e-6, eos_token_id=2, torch_dtype="bfloat16",
                    quantization_config={"quant_method": "fp8", "fmt": "e4m3", "activation_scheme": "dynamic",
                                         "weight_block_size": [128, 128]}),
    "tiny": dict(model_type="llama", hidden_size=1024, num_hidden_layers=2, num_attention_heads=8,
                 num_key_value_heads=2, head_dim=128, intermediate_size=2816, vocab_size=32000, rms_norm_eps=1e-5,
                 rope_theta=5e5, eos_token_id=2, torch_dtype="bfloat16"),
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--conc", type=int, default=256)
    ap.add_argument("--in-len", type=int, default=1024)
    ap.add_argument("--out-len", type=int, default=256)
    ap.add_argument("--batch-max-tokens", type=int, default=16384)
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--tpsp", action="store_true", help="token-sharded residual stream between layers (N > 1)")
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4, 5],
                    help="2 (default): Llama-3-8B, tensor parallel, fixed concurrency; 3: Llama-3-70B tensor parallel, "
                         "Poisson arrivals; 4: Qwen3-30B-A3B shapes, expert parallel; 5: DeepSeek-V3 shapes fp8, "
                         "data-parallel attention + expert parallel")
    ap.add_argument("--requests", type=int, default=None, help="config 3: number of requests (1000)")
    ap.add_argument("--rate", type=float, default=8.0, help="config 3: Poisson arrival rate, requests per second")
    ap.add_argument("--in-range", default="128,4096", help="config 3: uniform prompt length range")
    ap.add_argument("--out-range", default="64,1024", help="config 3: uniform output length range")
    ap.add_argument("--layers", type=int, default=None,
                    help="development aid: build only this many layers (the result line says so and is not a "
                         "measurement of the named configuration)")
    ap.add_argument("--warmup-out-len", type=int, default=None,
                    help="configs 3-5: output length of the warm-up runs (default 16: graph capture and first-use "
                         "set-up only; the timed runs use the configuration's lengths)")
    a = ap.parse_args()
    explicit = {x.split("=")[0] for x in sys.argv[1:] if x.startswith("--")}
    preset = {3: dict(model="llama3-70b", conc=256, batch_max_tokens=16384),
              4: dict(model="qwen3-30b-a3b", conc=512, in_len=2048, out_len=512, batch_max_tokens=8192),
              5: dict(model="deepseek-v3", conc=1024, in_len=1024, out_len=1024, batch_max_tokens=8192)}.get(a.config, {})
    for k, v in preset.items():
        if "--" + k.replace("_", "-") not in explicit:
            setattr(a, k, v)
    return a


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = f"/tmp/llb_clocks_{os.getpid()}.csv"
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)], stdout=self.f,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9:
                    continue
                sm.append(float(p[1]))
                mx.append(float(p[2]))
                for n, v in zip(names, p[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.remove(self.path)
        except Exception:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [s for s in sm if s >= 0.5 * max(sm)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def bench_config(args) -> dict:
    """The `config` entry of the result line; both arms print exactly this."""
    return {"model": args.model, "global_batch": args.conc, "seq_len": args.in_len + args.out_len,
            "input_len": args.in_len, "output_len": args.out_len,
            "parallelism": f"tp{args.gpus}" + ("+tpsp" if getattr(args, "tpsp", False) else ""),
            "batch_max_tokens": args.batch_max_tokens,
            "step": "one wave of `global_batch` requests: chunked prefill passes, all decode steps, greedy sampling",
            "l2": "inputs larger than L2 (weights and KV pool are streamed every pass)"}


def reference_arm(args):
    """The unmodified reference engine (installed under baseline/_ref) on the same workload."""
    try:
        from baseline import reference_runner  # noqa: WPS433
    except Exception as e:  # pragma: no cover
        print(json.dumps({"impl": "reference", "unavailable": f"reference runner not importable: {e}"[:300]}))
        return
    reference_runner.main(args, MODELS)


def serving_config(args, world):
    """Configurations 3 - 5, all through the public offline API `LLM.generate` (admission queue, radix cache,
    per-pass H2D of indices / prompt ids from pinned memory, per-pass D2H of the sampled ids, stop checks).

    3: Llama-3-70B shapes, tensor parallel over the N GPUs; `--requests` (1000) random-token requests, prompt length
       uniform in `--in-range`, output length uniform in `--out-range`, Poisson arrivals at `--rate` per second,
       seed 0.  One step = the whole arrival trace.  value = output tokens / time from the first arrival to the
       last token.
    4 / 5: Qwen3-30B-A3B / DeepSeek-V3 (fp8 block-scaled) shapes, data-parallel attention (one replica per GPU)
       with expert-parallel MoE; fixed input / output length; one step = one wave of `--conc` concurrent requests
       (conc / N per GPU).
    The device-timed value brackets the timed runs with CUDA events on the launching stream; the e2e value is the
    host clock around the same calls."""
    import torch

    from lightllm_b200 import ops
    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.parallel import dist as pdist

    moe = args.config in (4, 5)
    ps = pdist.init_from_env(dp=world if moe else 1)
    dev, rank = ps.device, ps.global_rank
    cuda = dev.type == "cuda"
    cfg = dict(MODELS[args.model])
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    t_start = time.time()

    def stage(msg):
        if rank == 0:
            print(f"[bench +{time.time() - t_start:6.1f}s] {msg}", file=sys.stderr, flush=True)

    rng = np.random.default_rng(0)
    vocab = cfg["vocab_size"]
    lo_id, hi_id = (1000, vocab - 1000) if vocab > 4000 else (3, vocab - 1)
    if args.config == 3:
        n_req = args.requests or 1000
        i0, i1 = (int(x) for x in args.in_range.split(","))
        o0, o1 = (int(x) for x in args.out_range.split(","))
        in_lens = rng.integers(i0, i1 + 1, size=n_req)
        out_lens = rng.integers(o0, o1 + 1, size=n_req)
        arrivals = np.cumsum(rng.exponential(1.0 / args.rate, size=n_req))
        arrivals -= arrivals[0]
        prompts = [rng.integers(lo_id, hi_id, size=int(n)).tolist() for n in in_lens]
        max_total = int(i1 + o1) + 8
        conc = args.conc
        pool = min(int(conc * (i1 + o1) * 0.6) + args.batch_max_tokens, conc * max_total)
        llm = LLM(config=cfg, max_total_token_num=pool, running_max_req_size=conc, max_req_total_len=max_total,
                  batch_max_tokens=args.batch_max_tokens, chunked_prefill_size=args.batch_max_tokens // 2,
                  graph_max_batch_size=conc)
        per_rank_conc = conc
    else:
        per_rank_conc = max(1, args.conc // world)
        total_len = args.in_len + args.out_len
        pool = per_rank_conc * (total_len + 8) + args.batch_max_tokens
        llm = LLM(config=cfg, max_total_token_num=pool, running_max_req_size=per_rank_conc,
                  max_req_total_len=total_len + 8, batch_max_tokens=args.batch_max_tokens,
                  chunked_prefill_size=args.batch_max_tokens // 2, graph_max_batch_size=per_rank_conc,
                  enable_ep_moe=world > 1)
    stage("model built")
    llm.warmup([per_rank_conc])
    stage("decode graph captured")

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        if cuda:
            torch.cuda.synchronize(dev)

    wrng = np.random.default_rng(1000 + rank)
    wlen = args.warmup_out_len or 16

    def one_run(warm: bool):
        """(output tokens of this rank, outs)"""
        if args.config == 3:
            if warm:   # a short burst of the same traffic
                k = min(32, len(prompts))
                sp = [{"max_new_tokens": wlen, "ignore_eos": True} for _ in range(k)]
                outs = llm.generate(prompts[:k], sp, arrival_times=list(arrivals[:k] * 0.1))
            else:
                sp = [{"max_new_tokens": int(o), "ignore_eos": True} for o in out_lens]
                outs = llm.generate(prompts, sp, return_stats=True, arrival_times=list(arrivals))[0]
            return sum(len(o["token_ids"]) for o in outs), outs
        n_here = max(1, per_rank_conc // 8) if warm else per_rank_conc
        ps_ = wrng.integers(lo_id, hi_id, size=(n_here, args.in_len)).tolist()
        sp = {"max_new_tokens": wlen if warm else args.out_len, "ignore_eos": True}
        outs = llm.generate(ps_, sp, return_stats=not warm)
        outs = outs[0] if not warm else outs
        return sum(len(o["token_ids"]) for o in outs), outs

    for i in range(args.warmup):
        one_run(True)
        if i == 0:
            stage("first warm-up run done")
    barrier()
    stage("warm-up done")
    clocks = ClockSampler(dev.index or 0)
    clocks.start()
    n0 = ops.launch_count()
    st0 = dict(llm.backend.stats)
    if cuda:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
    t0 = time.time()
    tokens, ttfts, itls = 0, [], []
    for _ in range(args.steps):
        n_tok, outs = one_run(False)
        tokens += n_tok
        for o in outs:
            if o["ttft_s"] is not None:
                ttfts.append(o["ttft_s"])
            tt = o.get("token_times") or []
            if len(tt) > 1:
                itls.append((tt[-1] - tt[0]) / (len(tt) - 1))
    if cuda:
        ev1.record()
    barrier()
    wall = time.time() - t0
    dev_ms = ev0.elapsed_time(ev1) if cuda else wall * 1e3
    launches = ops.launch_count() - n0
    clock_info = clocks.stop()
    st1 = llm.backend.stats
    fwd = (st1["prefill_steps"] - st0["prefill_steps"]) + (st1["decode_steps"] - st0["decode_steps"])
    h2d = (st1["h2d_bytes"] - st0["h2d_bytes"]) / max(fwd, 1)
    d2h = (st1["d2h_bytes"] - st0["d2h_bytes"]) / max(fwd, 1)
    status = int(ops.gemm_status(dev).item()) if cuda else 0
    v = torch.tensor([dev_ms, wall], dtype=torch.float64, device=dev)
    tk = torch.tensor([tokens if (moe or rank == 0) else 0], dtype=torch.float64, device=dev)
    lat = torch.tensor([statistics.median(ttfts) if ttfts else 0.0, statistics.median(itls) if itls else 0.0],
                       dtype=torch.float64, device=dev)
    if world > 1:
        torch.distributed.all_reduce(v, op=torch.distributed.ReduceOp.MAX)
        torch.distributed.all_reduce(tk)                                       # replicas serve different requests
        torch.distributed.all_reduce(lat, op=torch.distributed.ReduceOp.MAX)   # the slowest replica's medians
    dev_ms, wall, total_tokens = float(v[0]), float(v[1]), float(tk[0])
    if rank == 0:
        conf = bench_config(args)
        if args.config == 3:
            conf.update({"parallelism": f"tp{world}", "requests": len(prompts), "arrivals": f"Poisson {args.rate}/s, seed 0",
                         "input_len": f"uniform {args.in_range}", "output_len": f"uniform {args.out_range}",
                         "seq_len": max_total - 8, "global_batch": conc,
                         "step": "the whole arrival trace, first arrival to last token"})
        else:
            conf.update({"parallelism": f"dp{world}+ep{world}" if world > 1 else "single GPU",
                         "step": "one wave of `global_batch` concurrent requests (global_batch / N per GPU)",
                         "weights": "e4m3 with 128x128 block scales" if args.config == 5 else "bf16"})
        if "decode_gpu_ms" in st1:
            conf["decode_pass_device_ms"] = round((st1["decode_gpu_ms"] - st0.get("decode_gpu_ms", 0.0)) /
                                                  max(st1["decode_steps"] - st0["decode_steps"], 1), 3)
        steps_n = max(st1["decode_steps"] - st0["decode_steps"], 1)
        for key, name in (("agree_s", "host_vote_ms_per_decode_pass"), ("wait_gpu_s", "host_wait_for_gpu_ms_per_decode_pass")):
            if key in st1:
                conf[name] = round((st1[key] - st0.get(key, 0.0)) * 1e3 / steps_n, 3)
        if args.layers:
            conf["layers_override"] = f"{args.layers} layers only: NOT the named configuration"
        conf["warmup_runs"] = (f"{args.warmup} short runs (output length {wlen}, an eighth of the requests) of the "
                               "same traffic: graph capture and first-use set-up; the timed runs use the full "
                               "lengths and request counts")
        line = {"metric": "output tok/s per box at fixed concurrency" if moe else
                "output tok/s per box under Poisson arrivals", "value": round(total_tokens / (dev_ms / 1e3), 1),
                "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": round(dev_ms / args.steps, 2), "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "fp8 e4m3 weights / bf16 activations" if args.config == 5 else "bf16",
                "data": "synthetic uniform-random token ids, random-init weights", "impl": "ours", "config": conf,
                "clocks": clock_info, "gpu_launches": launches, "device_wait_status": status,
                "e2e": {"value": round(total_tokens / wall, 1), "unit": "tokens/s", "h2d_bytes_per_step": round(h2d, 1),
                        "d2h_bytes_per_step": round(d2h, 1),
                        "bytes_are_per": "forward pass (prefill chunk or decode step)",
                        "p50_ttft_ms": round(float(lat[0]) * 1e3, 2), "p50_itl_ms": round(float(lat[1]) * 1e3, 3)}}
        print(json.dumps(line), flush=True)
    llm.close()
    epg = getattr(llm.model, "_ep_group", None)
    if epg is not None:
        epg.close()
    pdist.destroy(hard_exit_on_hang=True)


def main():
    args = parse()
    if args.impl == "reference":
        reference_arm(args)
        return
    import torch

    from lightllm_b200 import ops
    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.parallel import dist as pdist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run"
    if args.config != 2:
        return serving_config(args, world)
    ps = pdist.init_from_env()
    dev = ps.device
    rank = ps.global_rank
    cfg = dict(MODELS[args.model])
    conc, in_len, out_len = args.conc, args.in_len, args.out_len
    total_len = in_len + out_len
    pool_tokens = conc * (total_len + 8) + args.batch_max_tokens
    llm = LLM(config=cfg, max_total_token_num=pool_tokens, running_max_req_size=conc, max_req_total_len=total_len + 8,
              batch_max_tokens=args.batch_max_tokens, chunked_prefill_size=args.batch_max_tokens // 2,
              disable_dynamic_prompt_cache=False, graph_max_batch_size=conc, tpsp_mix_mode=bool(args.tpsp))
    model = llm.model
    t_start = time.time()

    def stage(msg):  # progress on stderr (rank 0), so a slow stage shows up in the log of a cut-off run
        if rank == 0:
            print(f"[bench +{time.time() - t_start:6.1f}s] {msg}", file=sys.stderr, flush=True)

    stage("model built")
    llm.warmup([conc])
    stage("decode graph captured")
    rng = np.random.default_rng(1234)

    def new_prompts():
        return rng.integers(1000, cfg["vocab_size"] - 1000, size=(conc, in_len), dtype=np.int64)

    sp = {"max_new_tokens": out_len, "ignore_eos": True, "do_sample": False}

    # ---------------- device-timed wave through the model runner ----------------
    per_pass = max(1, args.batch_max_tokens // in_len)
    req_ids = torch.arange(conc, dtype=torch.int32)

    cuda = dev.type == "cuda"
    pin = (lambda t: t.pin_memory()) if cuda else (lambda t: t)
    seq_all = pin(torch.arange(in_len, total_len, dtype=torch.int32).view(-1, 1).repeat(1, conc).contiguous())
    b_req = pin(req_ids.clone())
    prefill_meta = []
    for s in range(0, conc, per_pass):
        e = min(conc, s + per_pass)
        B = e - s
        prefill_meta.append((s, e, pin(req_ids[s:e].clone()), pin(torch.full((B,), in_len, dtype=torch.int32)),
                             pin(torch.zeros(B, dtype=torch.int32))))

    phase_events = []   # (wave start, prefill done, wave done) CUDA events of the timed waves

    def static_wave(prompts_np, mark=False):
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(3)] if (mark and cuda) else None
        if evs:
            evs[0].record()
        mm = model.mem_manager
        mm.free_all()
        slots = mm.alloc(conc * total_len).clone().view(conc, total_len)
        slots_t = pin(slots.t().contiguous())           # [position, request]
        ids_all = pin(torch.from_numpy(prompts_np))
        nxt = model.req_manager.req_to_next_token_ids
        tok = None
        for s, e, reqs_p, len_p, zero_p in prefill_meta:
            B = e - s
            mi = ModelInput(batch_size=B, total_token_num=B * in_len, max_kv_len=in_len, is_prefill=True,
                            b_req_idx=reqs_p, b_seq_len=len_p,
                            mem_indexes=pin(slots[s:e, :in_len].reshape(-1).contiguous()),
                            input_ids=ids_all[s:e].reshape(-1), b_ready_cache_len=zero_p, b_q_len=len_p,
                            max_q_len=in_len)
            out = model.forward(mi)
            tok, _ = ops.sample(out.logits_any)
            ops.scatter_next_token_(nxt, tok, dev_req[s:e])
        if evs:
            evs[1].record()
        for t in range(1, out_len):
            L = in_len + t
            mi = ModelInput(batch_size=conc, total_token_num=conc * L, max_kv_len=L, is_prefill=False, b_req_idx=b_req,
                            b_seq_len=seq_all[t], mem_indexes=slots_t[L - 1])
            out = model.forward(mi)
            tok, _ = ops.sample(out.logits_any)
            ops.scatter_next_token_(nxt, tok, dev_req)
        if evs:
            evs[2].record()
            phase_events.append(evs)
        return tok

    dev_req = req_ids.to(dev)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        if cuda:
            torch.cuda.synchronize(dev)

    class _HostEvent:  # CPU dry runs only
        def record(self):
            self.t = time.time()

        def elapsed_time(self, other):
            return (other.t - self.t) * 1e3

    for i in range(args.warmup):
        static_wave(new_prompts())
        if i == 0:
            barrier()
            stage("first warm-up wave done")
    barrier()
    stage("warm-up done")
    clocks = ClockSampler(dev.index or 0)
    clocks.start()
    n0 = ops.launch_count()
    ev0, ev1 = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) if cuda else \
        (_HostEvent(), _HostEvent())
    ev0.record()
    for _ in range(args.steps):
        static_wave(new_prompts(), mark=True)
    ev1.record()
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    phases = None
    if phase_events:
        pre = sum(a.elapsed_time(b) for a, b, _ in phase_events) / len(phase_events)
        dec = sum(b.elapsed_time(c) for _, b, c in phase_events) / len(phase_events)
        phases = {"prefill_ms_per_step": round(pre, 1), "decode_ms_per_step": round(dec, 1),
                  "ms_per_decode_pass": round(dec / max(out_len - 1, 1), 3),
                  "note": "rank 0, device time inside the timed waves"}
    stage(f"timed waves done: {dev_ms / args.steps:.1f} ms/wave")
    launches = ops.launch_count() - n0
    clock_info = clocks.stop()
    status = int(ops.gemm_status(dev).item()) if cuda else 0
    model.mem_manager.free_all()

    # ---------------- end to end through the public API ----------------
    e2e = None
    ttft_p50 = itl_p50 = None
    if not args.skip_e2e:
        h2d0 = d2h0 = 0
        for _ in range(min(args.warmup, 1)):
            llm.generate(new_prompts().tolist(), sp)
        barrier()
        st0 = dict(llm.backend.stats)
        t0 = time.time()
        ttfts, itls = [], []
        for _ in range(args.steps):
            outs, _ = llm.generate(new_prompts().tolist(), sp, return_stats=True)
            for o in outs:
                if o["ttft_s"] is not None:
                    ttfts.append(o["ttft_s"])
                tt = o["token_times"]
                if len(tt) > 1:
                    itls.append((tt[-1] - tt[0]) / (len(tt) - 1))
        barrier()
        e2e_s = time.time() - t0
        st1 = llm.backend.stats
        fwd = (st1["prefill_steps"] - st0["prefill_steps"]) + (st1["decode_steps"] - st0["decode_steps"])
        e2e = {"seconds": e2e_s, "h2d": (st1["h2d_bytes"] - st0["h2d_bytes"]) / max(fwd, 1),
               "d2h": (st1["d2h_bytes"] - st0["d2h_bytes"]) / max(fwd, 1)}
        ttft_p50 = statistics.median(ttfts) * 1e3 if ttfts else None
        itl_p50 = statistics.median(itls) * 1e3 if itls else None

    # ---------------- max over ranks, print ----------------
    vals = torch.tensor([dev_ms, e2e["seconds"] if e2e else 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        torch.distributed.all_reduce(vals, op=torch.distributed.ReduceOp.MAX)
    dev_ms, e2e_s = float(vals[0]), float(vals[1])
    out_tokens = args.steps * conc * out_len
    value = out_tokens / (dev_ms / 1e3)
    if rank == 0:
        line = {
            "metric": "output tok/s per box at fixed concurrency", "value": round(value, 1), "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dev_ms / args.steps, 2), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
            "impl": "ours",
            "config": bench_config(args),
            "clocks": clock_info, "gpu_launches": launches, "device_wait_status": status, "phases": phases,
        }
        if e2e:
            line["e2e"] = {"value": round(out_tokens / e2e_s, 1), "unit": "tokens/s",
                           "h2d_bytes_per_step": round(e2e["h2d"], 1), "d2h_bytes_per_step": round(e2e["d2h"], 1),
                           "bytes_are_per": "forward pass (prefill chunk or decode step)",
                           "p50_ttft_ms": round(ttft_p50, 2) if ttft_p50 else None,
                           "p50_itl_ms": round(itl_p50, 3) if itl_p50 else None}
        print(json.dumps(line), flush=True)
    llm.close()
    pdist.destroy(hard_exit_on_hang=True)


if __name__ == "__main__":
    main()
