"""Decode steps launched ahead of the previous step's host bookkeeping give the same tokens as the synchronous
loop: length limits, end tokens (the extra token of a request that just ended is dropped), continuous batching."""
import os

import torch


def _llm(overlap: bool):
    from lightllm_b200.engine.llm import LLM

    cfg = dict(model_type="llama", hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, rms_norm_eps=1e-5, vocab_size=64, eos_token_id=7)
    llm = LLM(config=cfg, max_total_token_num=4096, running_max_req_size=8, max_req_total_len=256,
              batch_max_tokens=128, data_type="float32", eos_ids=tuple(range(16)))
    llm.backend.args.enable_decode_overlap = overlap
    return llm


def test_overlapped_decode_matches_synchronous_loop(monkeypatch):
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(16, 64, (n,), generator=g).tolist() for n in (5, 40, 17, 9, 70, 3)]
    params = [{"max_new_tokens": k} for k in (1, 2, 30, 13, 7, 40)]   # a small vocabulary: some hit the end token
    monkeypatch.delenv("LLB_FORCE_DECODE_OVERLAP", raising=False)
    want = _llm(False).generate(prompts, params)
    monkeypatch.setenv("LLB_FORCE_DECODE_OVERLAP", "1")
    llm = _llm(True)
    deferred = {"n": 0}
    orig = llm.backend._flush_pending

    def counting():
        if llm.backend._pending is not None:
            deferred["n"] += 1
        orig()

    llm.backend._flush_pending = counting
    got = llm.generate(prompts, params)
    assert deferred["n"] > 10, "the deferred path did not run"
    for a, b in zip(want, got):
        assert a["token_ids"] == b["token_ids"] and a["finish_reason"] == b["finish_reason"]
    assert any(o["finish_reason"] == "stop" for o in want) and any(o["finish_reason"] == "length" for o in want)
    assert llm.backend._pending is None and not llm.backend.ctx.requests
    # nothing leaked: every pool slot is either free or held by the prefix tree, and nothing is referenced
    rc = llm.backend.radix_cache
    assert llm.model.mem_manager.can_use_mem_size + rc.get_tree_total_tokens_num() == 4096
    assert rc.get_refed_tokens_num() == 0
