"""Sampling controls applied on the host side of a step (penalties, forbidden tokens) and the scheduler under
KV-pool pressure (requests are paused, re-prefilled later, and still produce what they produce with a large pool)."""
import numpy as np

from lightllm_b200.engine.llm import LLM

CFG = dict(model_type="llama", hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, vocab_size=300, rms_norm_eps=1e-5, eos_token_id=2)
KW = dict(running_max_req_size=8, max_req_total_len=256, batch_max_tokens=128, data_type="float32")


def test_repetition_penalty_and_forbidden_tokens():
    llm = LLM(config=CFG, max_total_token_num=4096, **KW)
    rng = np.random.default_rng(0)
    prompt = rng.integers(3, 300, 30).tolist()
    base = llm.generate([prompt], {"max_new_tokens": 24, "ignore_eos": True})[0]["token_ids"]
    pen = llm.generate([prompt], {"max_new_tokens": 24, "ignore_eos": True, "repetition_penalty": 50.0,
                                  "presence_penalty": 2.0, "frequency_penalty": 2.0})[0]["token_ids"]
    assert len(set(pen)) == len(pen)                       # nothing is said twice
    assert len(set(pen)) >= len(set(base))
    banned = llm.generate([prompt], {"max_new_tokens": 4, "ignore_eos": True,
                                     "invalid_token_ids": [base[0]]})[0]["token_ids"]
    assert banned[0] != base[0] and base[0] not in banned


def test_requests_paused_under_memory_pressure_finish_with_the_same_tokens():
    rng = np.random.default_rng(1)
    prompts = [rng.integers(3, 300, n).tolist() for n in (40, 35, 50, 45, 30, 38)]
    sp = {"max_new_tokens": 60, "ignore_eos": True}
    want = [o["token_ids"] for o in LLM(config=CFG, max_total_token_num=4096, **KW).generate(prompts, sp)]
    tight = LLM(config=CFG, max_total_token_num=330, **KW)       # all six together would need about 600 slots
    got = [o["token_ids"] for o in tight.generate(prompts, sp)]
    assert got == want
    st = tight.backend.stats
    mm, rc = tight.model.mem_manager, tight.backend.radix_cache
    assert mm.can_use_mem_size + rc.get_tree_total_tokens_num() == mm.size      # nothing leaked on the way


def test_backend_pauses_and_recovers_when_the_pool_runs_dry():
    """All requests are handed to the backend at once (no admission control): decode steps exhaust the pool, some
    requests give their KV back and re-prefill later; every request still ends with the tokens of a roomy run."""
    rng = np.random.default_rng(2)
    prompts = [rng.integers(3, 300, n).tolist() for n in (40, 35, 50, 45)]
    sp = {"max_new_tokens": 50, "ignore_eos": True}
    want = [o["token_ids"] for o in LLM(config=CFG, max_total_token_num=4096, **KW).generate(prompts, sp)]
    llm = LLM(config=CFG, max_total_token_num=260, **KW)          # prompts fit (170 + spare), the outputs do not
    llm.backend.args.pause_recover_interval = 4
    reqs = [llm._new_req(p, dict(sp)) for p in prompts]
    llm.backend.add_reqs(reqs)
    for _ in range(2000):
        if not llm.backend.has_work():
            break
        llm.backend.step()
    assert [r.get_output_ids() for r in reqs] == want
    assert llm.backend.stats["paused"] > 0
    mm, rc = llm.model.mem_manager, llm.backend.radix_cache
    assert mm.can_use_mem_size + rc.get_tree_total_tokens_num() == mm.size and rc.get_refed_tokens_num() == 0
