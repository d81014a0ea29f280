"""Tensor-parallel plumbing on CPU/gloo: TP=2 must reproduce TP=1 (tiny Llama, fp32, greedy)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

TINY = dict(model_type="llama", hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
            head_dim=64, intermediate_size=688, vocab_size=1024, rms_norm_eps=1e-6, rope_theta=1e4, eos_token_id=2)


def _prompts():
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(16, 65, (8,), generator=g).tolist()
    return [torch.randint(3, 1024, (n,), generator=g).tolist() for n in lens]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.parallel import dist as pdist

    torch.set_num_threads(2)
    pdist.init_distributed(world, rank, host="127.0.0.1", port=port, backend="gloo", device=torch.device("cpu"))
    llm = LLM(config=TINY, data_type="float32", max_total_token_num=4096, running_max_req_size=8,
              max_req_total_len=128, batch_max_tokens=256, random_seed=0)
    prompts = _prompts()
    # logits of one prefill pass
    m = llm.model
    ids = torch.tensor(prompts[0])
    req = m.req_manager.alloc()
    slots = m.mem_manager.alloc(len(ids))
    mi = ModelInput(batch_size=1, total_token_num=len(ids), max_kv_len=len(ids), is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([len(ids)], dtype=torch.int32),
                    mem_indexes=slots.clone(), input_ids=ids, b_ready_cache_len=torch.zeros(1, dtype=torch.int32),
                    max_q_len=len(ids))
    logits = m.forward(mi).logits
    m.mem_manager.free(slots)
    m.req_manager.free(req)
    outs = llm.generate(prompts, {"max_new_tokens": 32, "ignore_eos": True})
    if rank == 0:
        torch.save({"logits": logits, "tokens": [o["token_ids"] for o in outs]}, os.path.join(out_dir, f"tp{world}.pt"))
    pdist.destroy()


@pytest.mark.timeout(600)
def test_tp2_matches_tp1(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(1, port, str(tmp_path)), nprocs=1, join=True)
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a = torch.load(tmp_path / "tp1.pt")
    b = torch.load(tmp_path / "tp2.pt")
    assert a["logits"].shape == b["logits"].shape == (1, 1024)
    assert torch.allclose(a["logits"], b["logits"], atol=2e-4, rtol=1e-4), (a["logits"] - b["logits"]).abs().max()
    assert all(len(t) == 32 for t in b["tokens"])
    assert a["tokens"] == b["tokens"]


MOE = dict(model_type="qwen3_moe", hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
           head_dim=64, intermediate_size=688, moe_intermediate_size=128, num_experts=8, num_experts_per_tok=2,
           norm_topk_prob=True, vocab_size=1024, rms_norm_eps=1e-6, rope_theta=1e4, eos_token_id=2)


def _moe_worker(rank, world, port, out_dir, ep):
    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.parallel import dist as pdist

    torch.set_num_threads(2)
    pdist.init_distributed(world, rank, host="127.0.0.1", port=port, backend="gloo", device=torch.device("cpu"))
    llm = LLM(config=MOE, data_type="float32", max_total_token_num=2048, running_max_req_size=4,
              max_req_total_len=128, batch_max_tokens=128, enable_ep_moe=ep)
    outs = llm.generate(_prompts()[:4], {"max_new_tokens": 12, "ignore_eos": True})
    if rank == 0:
        torch.save([o["token_ids"] for o in outs], os.path.join(out_dir, f"moe_tp{world}_ep{int(ep)}.pt"))
    pdist.destroy()


@pytest.mark.timeout(600)
def test_moe_tp2_and_ep2_match_tp1(tmp_path):
    for world, ep in ((1, False), (2, False), (2, True)):
        mp.spawn(_moe_worker, args=(world, _free_port(), str(tmp_path), ep), nprocs=world, join=True)
    base = torch.load(tmp_path / "moe_tp1_ep0.pt")
    assert torch.load(tmp_path / "moe_tp2_ep0.pt") == base   # experts sliced along the intermediate dim
    assert torch.load(tmp_path / "moe_tp2_ep1.pt") == base   # whole experts per rank


NEW_FAMILIES = {
    "gemma4_text": dict(model_type="gemma4_text", hidden_size=128, intermediate_size=256, num_hidden_layers=4,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=32, global_head_dim=64,
                        sliding_window=16, layer_types=["sliding_attention", "full_attention", "sliding_attention",
                                                        "full_attention"],
                        num_kv_shared_layers=2, use_double_wide_mlp=True, hidden_size_per_layer_input=16,
                        vocab_size_per_layer_input=512, enable_moe_block=True, num_experts=4, top_k_experts=2,
                        moe_intermediate_size=64, vocab_size=512, eos_token_id=2, tie_word_embeddings=True),
    "qwen3_5_text": dict(model_type="qwen3_5_text", hidden_size=128, intermediate_size=256, num_hidden_layers=4,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=32, vocab_size=512, rms_norm_eps=1e-6,
                         linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=16,
                         linear_value_head_dim=16, linear_conv_kernel_dim=4, full_attention_interval=2,
                         eos_token_id=2, tie_word_embeddings=False),
    "deepseek_v32": dict(model_type="deepseek_v32", hidden_size=128, intermediate_size=256, moe_intermediate_size=64,
                         num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4, n_routed_experts=4,
                         n_shared_experts=1, num_experts_per_tok=2, n_group=2, topk_group=1, first_k_dense_replace=1,
                         q_lora_rank=32, kv_lora_rank=48, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                         vocab_size=512, routed_scaling_factor=2.5, norm_topk_prob=True, rms_norm_eps=1e-6,
                         index_n_heads=4, index_head_dim=16, index_topk=12, eos_token_id=2),
}


def _family_worker(rank, world, port, out_dir, family):
    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.parallel import dist as pdist

    torch.set_num_threads(2)
    pdist.init_distributed(world, rank, host="127.0.0.1", port=port, backend="gloo", device=torch.device("cpu"))
    llm = LLM(config=NEW_FAMILIES[family], data_type="float32", max_total_token_num=2048, running_max_req_size=4,
              max_req_total_len=128, batch_max_tokens=128, random_seed=0)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(3, 512, (n,), generator=g).tolist() for n in (20, 45, 33)]
    outs = llm.generate(prompts, {"max_new_tokens": 12, "ignore_eos": True})
    if rank == 0:
        torch.save({"tokens": [o["token_ids"] for o in outs], "logprobs": [o["logprobs"] for o in outs]},
                   os.path.join(out_dir, f"{family}_tp{world}.pt"))
    pdist.destroy()


@pytest.mark.timeout(900)
@pytest.mark.parametrize("family", sorted(NEW_FAMILIES))
def test_newer_families_tp2_matches_tp1(tmp_path, family):
    for world in (1, 2):
        mp.spawn(_family_worker, args=(world, _free_port(), str(tmp_path), family), nprocs=world, join=True)
    a = torch.load(tmp_path / f"{family}_tp1.pt")
    b = torch.load(tmp_path / f"{family}_tp2.pt")
    la, lb = np.concatenate(a["logprobs"]), np.concatenate(b["logprobs"])
    assert a["tokens"] == b["tokens"] or np.abs(la - lb).max() < 5e-3
    assert np.abs(la[:3] - lb[:3]).max() < 1e-3          # the first tokens of the first request agree closely


def _abort_worker(rank, world, port, out_dir):
    """The HTTP worker raises `is_aborted` in the shared request at an arbitrary moment; tensor-parallel ranks
    whose loops are a step apart see it at different steps.  Only the abort command (delivered to all ranks at
    the same point of their schedules) may drop the request."""
    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.parallel import dist as pdist

    torch.set_num_threads(2)
    pdist.init_distributed(world, rank, host="127.0.0.1", port=port, backend="gloo", device=torch.device("cpu"))
    llm = LLM(config=TINY, data_type="float32", max_total_token_num=4096, running_max_req_size=8,
              max_req_total_len=128, batch_max_tokens=256, random_seed=0)
    be = llm.backend
    reqs = [llm._new_req(p, {"max_new_tokens": 12, "ignore_eos": True}) for p in _prompts()[:3]]
    be.add_reqs(reqs)
    victim = reqs[1]
    log = []
    for step in range(40):
        if not be.has_work():
            break
        if step == 3 + rank:               # rank 0 sees the flag one step earlier than rank 1
            victim.is_aborted = True
        if step == 6:                      # the command reaches both ranks at the same step
            be.abort(victim.request_id)
        res = be.step()
        log.append((res["kind"], res["tokens"], sorted(r.req_id for r in res["finished"])))
    torch.save({"log": log, "tokens": [r.get_output_ids() for r in reqs],
                "reasons": [r.finish_status.get_finish_reason() for r in reqs]},
               os.path.join(out_dir, f"abort_rank{rank}.pt"))
    pdist.destroy()


@pytest.mark.timeout(600)
def test_abort_flag_seen_at_different_steps_keeps_ranks_in_step(tmp_path):
    mp.spawn(_abort_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    a, b = torch.load(tmp_path / "abort_rank0.pt"), torch.load(tmp_path / "abort_rank1.pt")
    assert a["log"] == b["log"]                      # identical schedules, step by step
    assert a["tokens"] == b["tokens"]
    assert a["reasons"][1] == "abort" and a["reasons"][0] == a["reasons"][2] == "length"
    kinds = [k for k, _, _ in a["log"]]
    first_without = next(i for i, (_, _, fin) in enumerate(a["log"]) if fin)
    assert first_without == 6                        # dropped on the step of the command, not of the flag
    assert len(a["tokens"][0]) == 12 and "decode" in kinds
