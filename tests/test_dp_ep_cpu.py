"""Data-parallel attention with expert-parallel MoE on CPU/gloo (world 2, dp 2): every rank serves its own
prompts, the ranks step in lock-step (the idle one holds), tokens travel to the experts' ranks and back; the
outputs equal a single-process run."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

CFG = dict(model_type="qwen3_moe", hidden_size=128, intermediate_size=256, moe_intermediate_size=64,
           num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32, num_experts=8,
           num_experts_per_tok=2, norm_topk_prob=True, vocab_size=512, rms_norm_eps=1e-6, eos_token_id=2,
           decoder_sparse_step=1, mlp_only_layers=[])
DS = dict(model_type="deepseek_v3", hidden_size=128, intermediate_size=256, moe_intermediate_size=64,
          num_hidden_layers=2, num_attention_heads=4, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2,
          n_group=2, topk_group=1, first_k_dense_replace=1, q_lora_rank=32, kv_lora_rank=48, qk_nope_head_dim=16,
          qk_rope_head_dim=8, v_head_dim=16, vocab_size=512, routed_scaling_factor=2.5, norm_topk_prob=True,
          rms_norm_eps=1e-6, eos_token_id=2)


def _prompts():
    g = torch.Generator().manual_seed(3)
    return [torch.randint(3, 512, (n,), generator=g).tolist() for n in (21, 40, 9, 33, 17)]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, dp, port, out_dir, cfg):
    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.parallel import dist as pdist

    torch.set_num_threads(2)
    pdist.init_distributed(world, rank, dp=dp, host="127.0.0.1", port=port, backend="gloo", device=torch.device("cpu"))
    llm = LLM(config=cfg, data_type="float32", max_total_token_num=4096, running_max_req_size=8, max_req_total_len=128,
              batch_max_tokens=64, random_seed=0, enable_ep_moe=world > 1)
    prompts = _prompts()
    mine = prompts if world == 1 else (prompts[:4] if rank == 0 else prompts[4:])   # 4 requests vs 1: the ranks go idle apart
    outs = llm.generate(mine, {"max_new_tokens": 12, "ignore_eos": True})
    torch.save({"tokens": [o["token_ids"] for o in outs], "stats": dict(llm.backend.stats)},
               os.path.join(out_dir, f"w{world}_r{rank}.pt"))
    pdist.destroy()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("name", ["qwen3_moe", "deepseek_v3"])
def test_dp2_ep2_matches_single(tmp_path, name):
    cfg = CFG if name == "qwen3_moe" else DS
    mp.spawn(_worker, args=(1, 1, _free_port(), str(tmp_path), cfg), nprocs=1, join=True)
    mp.spawn(_worker, args=(2, 2, _free_port(), str(tmp_path), cfg), nprocs=2, join=True)
    one = torch.load(tmp_path / "w1_r0.pt")
    r0, r1 = torch.load(tmp_path / "w2_r0.pt"), torch.load(tmp_path / "w2_r1.pt")
    assert r0["tokens"] == one["tokens"][:4]
    assert r1["tokens"] == one["tokens"][4:]
    assert r1["stats"]["hold_prefill"] + r1["stats"]["hold_decode"] > 0   # the short rank kept stepping for the other


def _worker_tp_in_replica(rank, world, dp, port, out_dir):
    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.parallel import dist as pdist

    torch.set_num_threads(1)
    ps = pdist.init_distributed(world, rank, dp=dp, host="127.0.0.1", port=port, backend="gloo",
                                device=torch.device("cpu"))
    llm = LLM(config=CFG, data_type="float32", max_total_token_num=4096, running_max_req_size=8, max_req_total_len=128,
              batch_max_tokens=64, random_seed=0, enable_ep_moe=True)
    prompts = _prompts()
    mine = prompts[:4] if ps.dp_rank == 0 else prompts[4:]
    outs = llm.generate(mine, {"max_new_tokens": 12, "ignore_eos": True})
    lw = llm.model.layers[0]
    torch.save({"tokens": [o["token_ids"] for o in outs], "experts": tuple(lw.w13.shape), "e0": lw.e0},
               os.path.join(out_dir, f"tpdp_r{rank}.pt"))
    pdist.destroy()


@pytest.mark.timeout(900)
def test_dp2_with_tp2_replicas_and_ep4_matches_single(tmp_path):
    """4 ranks: 2 replicas of 2 tensor-parallel ranks each, the 8 experts spread over all 4 ranks."""
    mp.spawn(_worker, args=(1, 1, _free_port(), str(tmp_path), CFG), nprocs=1, join=True)
    mp.spawn(_worker_tp_in_replica, args=(4, 2, _free_port(), str(tmp_path)), nprocs=4, join=True)
    one = torch.load(tmp_path / "w1_r0.pt")
    rs = [torch.load(tmp_path / f"tpdp_r{r}.pt") for r in range(4)]
    assert rs[0]["tokens"] == one["tokens"][:4]       # a replica's first rank publishes its tokens
    assert rs[2]["tokens"] == one["tokens"][4:]
    assert [r["experts"][0] for r in rs] == [2, 2, 2, 2] and [r["e0"] for r in rs] == [0, 2, 4, 6]
