"""A saved prompt prefix (`prompt_cache_kv_buffer` + `prompt_cache_token_ids` in config.json): the KV rows written by
one engine are loaded and pinned by another at start-up; the first request with that prefix is a cache hit and
produces the same tokens.  Reference: lightllm/server/router/model_infer/mode_backend/base_backend.py:961-977."""
import pytest
import torch

CFG = dict(model_type="llama", hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
           head_dim=32, intermediate_size=256, vocab_size=512, rms_norm_eps=1e-6, rope_theta=10000.0, eos_token_id=2)
KW = dict(data_type="float32", max_total_token_num=1024, running_max_req_size=4, max_req_total_len=256,
          batch_max_tokens=128, random_seed=0)


def test_save_then_preload(tmp_path):
    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.parallel import dist as pdist

    pdist.init_distributed(1, 0, device=torch.device("cpu"))
    g = torch.Generator().manual_seed(4)
    system = torch.randint(3, 512, (70,), generator=g).tolist()
    question = torch.randint(3, 512, (15,), generator=g).tolist()
    sp = {"max_new_tokens": 6, "ignore_eos": True}
    a = LLM(config=CFG, **KW)
    want = a.generate([system + question], sp)[0]
    assert want["prompt_cache_len"] == 0
    path = tmp_path / "prompt_cache_rank_0.pt"
    assert a.backend.save_prompt_cache_kv(system, str(path)) == 70
    cfg = dict(CFG, prompt_cache_kv_buffer={"rank_0": str(path)}, prompt_cache_token_ids=system)
    b = LLM(config=cfg, **KW)
    assert b.backend.stats["prompt_cache_preloaded_tokens"] == 70
    free0 = b.model.mem_manager.can_use_mem_size
    got = b.generate([system + question], sp)[0]
    assert got["prompt_cache_len"] == 70 and got["token_ids"] == want["token_ids"]
    # pinned: flushing the cache does not drop it
    b.backend.radix_cache.clear_tree_nodes()
    assert b.generate([system + question[:5]], sp)[0]["prompt_cache_len"] == 70
    assert b.model.mem_manager.can_use_mem_size <= free0
    # a file for another pool layout is refused
    bad = dict(CFG, num_key_value_heads=4, prompt_cache_kv_buffer={"rank_0": str(path)}, prompt_cache_token_ids=system)
    with pytest.raises(ValueError):
        LLM(config=bad, **KW)
    pdist.destroy()
