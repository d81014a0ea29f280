"""Speculative decoding under lock-step data parallelism with expert parallelism (CPU / gloo, 2 replicas): every
replica runs the same sequence of passes per round (target pass + `mtp_step` draft passes, over the hold request when
it has nothing to do), so the MoE exchanges of target and draft modules line up although the replicas serve
different numbers of requests; the tokens are the target's plain greedy tokens.
Reference: lightllm/server/router/model_infer/mode_backend/dp_backend/impl.py (prefill_mtp / decode_mtp)."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

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


def _worker(rank, world, port, out_dir, k):
    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.models.mtp import build_mtp_modules
    from lightllm_b200.parallel import dist as pdist

    torch.set_num_threads(2)
    pdist.init_distributed(world, rank, dp=world, host="127.0.0.1", port=port, backend="gloo", device=torch.device("cpu"))
    llm = LLM(config=DS, data_type="float32", max_total_token_num=4096, running_max_req_size=8, max_req_total_len=128,
              batch_max_tokens=64, random_seed=0, enable_ep_moe=world > 1, extra_kv_layers=1 if k else 0)
    if k:
        from lightllm_b200.engine.mtp_backend import DPMTPBackend, MTPBackend

        drafts = build_mtp_modules(llm.model, 1)
        cls = DPMTPBackend if world > 1 else MTPBackend
        llm.backend = cls(llm.model, llm.args, draft_models=drafts, mtp_step=k, is_master_in_dp=True)
    prompts = _prompts()
    mine = prompts if world == 1 else (prompts[:4] if rank == 0 else prompts[4:])   # 4 requests against 1
    outs = llm.generate(mine, {"max_new_tokens": 14, "ignore_eos": True})
    torch.save({"tokens": [o["token_ids"] for o in outs], "stats": dict(llm.backend.stats)},
               os.path.join(out_dir, f"w{world}_r{rank}_k{k}.pt"))
    pdist.destroy()


@pytest.mark.timeout(900)
@pytest.mark.parametrize("k", [1, 2])
def test_dp2_ep2_mtp_matches_plain_greedy(tmp_path, k):
    mp.spawn(_worker, args=(1, _free_port(), str(tmp_path), 0), nprocs=1, join=True)
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), k), nprocs=2, join=True)
    one = torch.load(tmp_path / "w1_r0_k0.pt")
    r0, r1 = torch.load(tmp_path / f"w2_r0_k{k}.pt"), torch.load(tmp_path / f"w2_r1_k{k}.pt")
    assert r0["tokens"] == one["tokens"][:4] and r1["tokens"] == one["tokens"][4:]
    assert r0["stats"]["mtp_steps"] > 0 and r1["stats"]["mtp_steps"] > 0
    assert r1["stats"]["hold_prefill"] + r1["stats"]["hold_decode"] > 0      # the short replica kept in step
