"""`--enable_fused_shared_experts`: the shared expert of a DeepSeek-style MoE layer runs inside the grouped expert
GEMMs (as experts every token selects with weight 1) and gives the logits of the separate path; also under tensor
parallelism (2 gloo ranks).  Reference: lightllm/models/deepseek2/layer_weights/transformer_layer_weight.py
(`enable_fused_shared_experts`: shared experts appended to the routed ones)."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

DS = dict(model_type="deepseek_v3", hidden_size=128, intermediate_size=256, moe_intermediate_size=64,
          num_hidden_layers=2, num_attention_heads=4, n_routed_experts=8, n_shared_experts=2, num_experts_per_tok=2,
          n_group=2, topk_group=1, first_k_dense_replace=1, q_lora_rank=32, kv_lora_rank=48, qk_nope_head_dim=16,
          qk_rope_head_dim=8, v_head_dim=16, vocab_size=512, routed_scaling_factor=2.5, norm_topk_prob=True,
          rms_norm_eps=1e-6, eos_token_id=2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir, fused):
    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.parallel import dist as pdist

    torch.set_num_threads(2)
    pdist.init_distributed(world, rank, host="127.0.0.1", port=port, backend="gloo", device=torch.device("cpu"))
    llm = LLM(config=DS, data_type="float32", max_total_token_num=1024, running_max_req_size=4, max_req_total_len=128,
              batch_max_tokens=128, random_seed=0, enable_fused_shared_experts=fused)
    m = llm.model
    lw = m.layers[1]
    ids = torch.randint(3, 512, (40,), generator=torch.Generator().manual_seed(2))
    req = m.req_manager.alloc()
    mi = ModelInput(batch_size=1, total_token_num=40, max_kv_len=40, is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([40], dtype=torch.int32),
                    mem_indexes=m.mem_manager.alloc(40).clone(), input_ids=ids,
                    b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=40, return_all_logits=True)
    logits = m.forward(mi).logits.float()
    if rank == 0:
        torch.save({"logits": logits, "experts": lw.w13.shape[0], "fused": lw.fused_shared,
                    "has_shared": lw.shared_down_w is not None},
                   os.path.join(out_dir, f"w{world}_f{int(fused)}.pt"))
    pdist.destroy()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("world", [1, 2])
def test_fused_shared_experts_match_the_separate_path(tmp_path, world):
    for fused in (False, True):
        mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), fused), nprocs=world, join=True)
    a, b = torch.load(tmp_path / f"w{world}_f0.pt"), torch.load(tmp_path / f"w{world}_f1.pt")
    assert a["experts"] == 8 and a["fused"] == 0 and a["has_shared"]
    assert b["experts"] == 10 and b["fused"] == 2 and not b["has_shared"]
    scale = a["logits"].abs().max().item()
    assert (a["logits"] - b["logits"]).abs().max().item() < 1e-4 * scale
