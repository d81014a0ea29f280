"""Host (and disk) tier of the prefix cache on CPU: pages survive the eviction of the GPU prefix tree and give
the same continuation as an uncached run."""
import numpy as np
import torch

from lightllm_b200.engine.host_kv_cache import HostKVCache, page_keys
from lightllm_b200.engine.llm import LLM

CFG = dict(model_type="llama", hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, vocab_size=500, rms_norm_eps=1e-5, eos_token_id=2)


def test_page_keys_chain():
    a = page_keys(np.arange(100), 16)
    b = page_keys(np.concatenate([np.arange(48), np.arange(100, 152)]), 16)
    assert len(a) == 6 and a[:3] == b[:3] and a[3] != b[3]


def _llm(tmp_path=None, **kw):
    return LLM(config=CFG, max_total_token_num=2048, running_max_req_size=4, max_req_total_len=512, batch_max_tokens=512,
               data_type="float32", cpu_cache_bytes=4 << 20, cpu_cache_page_tokens=16, **kw)


def test_host_tier_serves_prefix_after_gpu_eviction(tmp_path):
    rng = np.random.default_rng(0)
    shared = rng.integers(3, 500, 70).tolist()
    p1, p2 = shared + [11, 12, 13], shared + [21, 22, 23, 24]
    sp = {"max_new_tokens": 6, "ignore_eos": True}
    base = LLM(config=CFG, max_total_token_num=2048, running_max_req_size=4, max_req_total_len=512, batch_max_tokens=512,
               data_type="float32")
    want = base.generate([p2], sp)[0]["token_ids"]

    llm = _llm()
    hc = llm.backend.ctx.host_cache
    assert isinstance(hc, HostKVCache)
    llm.generate([p1], sp)
    assert hc.stats["offloaded_pages"] == (len(p1) + 6 - 1) // 16    # every full page of prompt + output in the pool
    llm.backend.radix_cache.clear_tree_nodes()                        # the GPU tier forgets everything
    out = llm.generate([p2], sp)[0]
    assert out["token_ids"] == want
    assert hc.stats["loaded_pages"] == 4 and hc.stats["host_hits"] == 4   # 70 shared tokens = 4 full pages of 16


def test_disk_tier_takes_evicted_pages(tmp_path):
    rng = np.random.default_rng(1)
    sp = {"max_new_tokens": 2, "ignore_eos": True}
    llm = LLM(config=CFG, max_total_token_num=2048, running_max_req_size=4, max_req_total_len=512, batch_max_tokens=512,
              data_type="float32", cpu_cache_bytes=1, cpu_cache_page_tokens=16, disk_cache_dir=str(tmp_path),
              disk_cache_bytes=8 << 20)   # host tier of a single page: everything older goes to disk
    hc = llm.backend.ctx.host_cache
    assert hc.n_pages == 1 and hc.disk is not None
    prompt = rng.integers(3, 500, 50).tolist()
    first = llm.generate([prompt], sp)[0]["token_ids"]
    assert len(hc.disk.index) >= 2
    llm.backend.radix_cache.clear_tree_nodes()
    again = llm.generate([prompt], sp)[0]["token_ids"]
    assert again == first and hc.stats["disk_hits"] >= 2


def test_two_pool_cache_of_gemma4_moves_through_staging_pages():
    """Gemma-4 keeps two KV pools with different head sizes; staging pages carry a token's rows of both."""
    import numpy as np
    import torch

    from lightllm_b200.engine.llm import LLM

    cfg = dict(model_type="gemma4_text", hidden_size=64, intermediate_size=128, num_hidden_layers=3,
               num_attention_heads=4, num_key_value_heads=2, head_dim=16, global_head_dim=32, sliding_window=16,
               layer_types=["sliding_attention", "sliding_attention", "full_attention"], hidden_size_per_layer_input=0,
               vocab_size=300, eos_token_id=2, tie_word_embeddings=True)
    kw = dict(max_total_token_num=1024, running_max_req_size=4, max_req_total_len=256, batch_max_tokens=128,
              data_type="float32")
    llm = LLM(config=cfg, **kw)
    mm = llm.model.mem_manager
    assert mm.layer_num == 1 and mm.kv_row_shape() == (2 * 2 * 2 * 16 + 1 * 2 * 2 * 32,)
    mm.kv_sliding.normal_()
    mm.kv_global.normal_()
    src, dst = torch.tensor([3, 9, 40], dtype=torch.int32), torch.tensor([100, 7, 55], dtype=torch.int32)
    pages = mm.gather_pages(src)
    assert pages.shape == (1, 3, 256)
    mm.scatter_pages(dst, pages)
    assert torch.equal(mm.kv_sliding[:, dst.long()], mm.kv_sliding[:, src.long()])
    assert torch.equal(mm.kv_global[:, dst.long()], mm.kv_global[:, src.long()])
    # the host tier on top of it: a prompt evicted from the GPU tree comes back from host pages
    rng = np.random.default_rng(0)
    prompt = rng.integers(3, 300, 130).tolist()
    sp = {"max_new_tokens": 6, "ignore_eos": True}
    want = LLM(config=cfg, **kw).generate([prompt], sp)[0]["token_ids"]
    tiered = LLM(config=cfg, cpu_cache_bytes=4 << 20, cpu_cache_page_tokens=32, **kw)
    assert tiered.generate([prompt], sp)[0]["token_ids"] == want
    tiered.backend.radix_cache.free_radix_cache_to_get_enough_token(1024)         # drop the GPU copy
    again = tiered.generate([prompt], sp)[0]
    assert again["token_ids"] == want and tiered.backend.ctx.host_cache.stats["host_hits"] > 0
