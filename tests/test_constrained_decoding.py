"""Grammar-constrained decoding through xgrammar token bitmasks: whatever the (random) model prefers, the emitted
text matches the grammar and the request stops when the grammar is complete."""
import json

import numpy as np
import pytest
import torch

xgr = pytest.importorskip("xgrammar")

from lightllm_b200.engine.llm import LLM  # noqa: E402
from lightllm_b200.engine.mode_backends import XgrammarBackend  # noqa: E402

CFG = dict(model_type="llama", hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, vocab_size=300, rms_norm_eps=1e-5, eos_token_id=2)
KW = dict(max_total_token_num=2048, running_max_req_size=8, max_req_total_len=256, batch_max_tokens=128,
          data_type="float32")
VOCAB = ["<pad>", "<bos>", "<eos>"] + [chr(c) for c in range(32, 127)]
VOCAB += [f"<x{i}>" for i in range(300 - len(VOCAB))]


def _llm():
    llm = LLM(config=CFG, **KW)
    info = xgr.TokenizerInfo(VOCAB, vocab_type=xgr.VocabType.RAW, vocab_size=300, stop_token_ids=[2])
    llm.backend = XgrammarBackend(llm.model, llm.args, tokenizer_info=info, is_master_in_dp=True)
    return llm


def _text(ids):
    return "".join(VOCAB[i] for i in ids if i != 2)


def test_ebnf_grammar_shapes_the_output():
    llm = _llm()
    rng = np.random.default_rng(0)
    prompts = [rng.integers(3, 98, n).tolist() for n in (5, 17, 9)]
    grammar = 'root ::= ("yes" | "no") " " [0-9] [0-9] "!"'
    outs = llm.generate(prompts, {"max_new_tokens": 40, "guided_grammar": grammar})
    for o in outs:
        t = _text(o["token_ids"])
        head, tail = (t[:3], t[3:]) if t.startswith("yes") else (t[:2], t[2:])
        assert head in ("yes", "no") and tail[0] == " " and tail[1:3].isdigit() and tail[3] == "!" and len(tail) == 4
        assert o["finish_reason"] == "stop"
    # an unconstrained request in the same batch is left alone
    mixed = llm.generate(prompts[:2], [{"max_new_tokens": 6, "guided_grammar": grammar},
                                       {"max_new_tokens": 6, "ignore_eos": True}])
    assert len(mixed[1]["token_ids"]) == 6


def test_json_schema_constraint():
    llm = _llm()
    schema = {"enum": ["red", "green", 7]}
    outs = llm.generate([[5, 6, 7, 8], [9, 10]], {"max_new_tokens": 30, "guided_json": schema})
    for o in outs:
        assert json.loads(_text(o["token_ids"])) in ("red", "green", 7) and o["finish_reason"] == "stop"


def test_first_token_constraint(monkeypatch):
    from lightllm_b200.engine.mode_backends import FirstTokenConstraintBackend

    monkeypatch.setenv("FIRST_ALLOWED_TOKENS", "41,42,43")
    llm = LLM(config=CFG, **KW)
    llm.backend = FirstTokenConstraintBackend(llm.model, llm.args, is_master_in_dp=True)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(3, 300, n).tolist() for n in (5, 40, 9, 70)]
    outs = llm.generate(prompts, {"max_new_tokens": 5, "ignore_eos": True})
    plain = LLM(config=CFG, **KW).generate(prompts, {"max_new_tokens": 5, "ignore_eos": True})
    for o, p in zip(outs, plain):
        assert o["token_ids"][0] in (41, 42, 43) and len(o["token_ids"]) == 5
        assert p["token_ids"][0] not in (41, 42, 43)        # the unconstrained model says something else


def test_token_healing_regenerates_the_cut_text():
    """The prompt's last tokens were removed (their text is the prefix to heal): generation may only continue that
    text until it is covered, then runs free."""
    from lightllm_b200.engine.mode_backends import TokenHealingBackend

    class Tok:
        def convert_ids_to_tokens(self, ids):
            return [VOCAB[i] if 3 <= i < 98 else "" for i in ids]

    llm = LLM(config=CFG, **KW)
    llm.backend = TokenHealingBackend(llm.model, llm.args, tokenizer=Tok(), is_master_in_dp=True)
    cut = [VOCAB.index(c) for c in "hel"]
    req = llm._new_req([5, 6, 7, 8, 9], {"max_new_tokens": 6, "ignore_eos": True})
    req.prefix_token_ids.set(cut)
    llm.queue.extend([req])
    from lightllm_b200.server.router.req_queue import Batch

    running = Batch(0, [])
    for _ in range(50):
        nb = llm.queue.generate_new_batch(running)
        if nb is not None:
            llm.backend.add_reqs(nb.reqs)
            running.merge(nb)
        if not llm.backend.has_work():
            break
        llm.backend.step()
        running.filter_out_finished_req()
    text = _text(req.get_output_ids())
    assert text.startswith("hel") and len(req.get_output_ids()) == 6


def test_reward_backend_scores_prompts_without_decoding():
    from lightllm_b200.engine.mode_backends import RewardModelBackend

    cfg = dict(CFG, model_type="qwen2", architectures=["Qwen2ForRewardModel"])
    llm = LLM(config=cfg, **KW)
    assert "Reward" in type(llm.model).__name__
    llm.backend = RewardModelBackend(llm.model, llm.args, is_master_in_dp=True)
    rng = np.random.default_rng(2)
    a, b = rng.integers(3, 300, 20).tolist(), rng.integers(3, 300, 33).tolist()
    reqs = [llm._new_req(p, {"max_new_tokens": 1}) for p in (a, b, a)]
    llm.queue.extend(reqs)
    from lightllm_b200.server.router.req_queue import Batch

    running = Batch(0, [])
    for _ in range(20):
        nb = llm.queue.generate_new_batch(running)
        if nb is not None:
            llm.backend.add_reqs(nb.reqs)
            running.merge(nb)
        if not llm.backend.has_work():
            break
        llm.backend.step()
        running.filter_out_finished_req()
    s = [r.reward_score for r in reqs]
    assert all(np.isfinite(s)) and abs(s[0] - s[2]) < 1e-5 and abs(s[0] - s[1]) > 1e-6
    assert all(r.finish_status.is_finished() for r in reqs) and llm.backend.stats["decode_steps"] == 0


def test_diverse_backend_shares_the_prompt_between_samples():
    from lightllm_b200.engine.mode_backends import DiverseBackend

    llm = LLM(config=CFG, **KW)
    llm.backend = DiverseBackend(llm.model, llm.args, is_master_in_dp=True)
    prompt = np.random.default_rng(3).integers(3, 300, 60).tolist()
    group = [llm._new_req(prompt, {"max_new_tokens": 5, "ignore_eos": True, "do_sample": True, "temperature": 1.0,
                                   "top_k": 50, "seed": 10 + i}) for i in range(3)]
    for r in group:
        r.group_req_id = group[0].request_id
    llm.queue.extend(group)
    from lightllm_b200.server.router.req_queue import Batch

    running = Batch(0, [])
    for _ in range(60):
        nb = llm.queue.generate_new_batch(running)
        if nb is not None:
            llm.backend.add_reqs(nb.reqs)
            running.merge(nb)
        if not llm.backend.has_work() and not getattr(llm.backend, "_deferred", []):
            break
        llm.backend.step()
        running.filter_out_finished_req()
    assert all(len(r.get_output_ids()) == 5 for r in group)
    # the prompt was computed once: the siblings found all but its last token in the prefix tree
    assert llm.backend.stats["prefill_tokens"] <= 60 + 2 * 2
    assert [r.prompt_cache_len for r in group[1:]] == [59, 59]


def test_regular_expression_constraint_on_the_grammar_matcher():
    llm = _llm()
    outs = llm.generate([[5, 6, 7], [8, 9, 10, 11]], {"max_new_tokens": 30, "regular_constraint": r"[A-C]{2}-[0-9]{3}"})
    import re

    for o in outs:
        assert re.fullmatch(r"[A-C]{2}-[0-9]{3}", _text(o["token_ids"])) and o["finish_reason"] == "stop"


def test_prompt_logprobs_match_a_direct_forward_pass():
    from lightllm_b200.common.infer_state import ModelInput

    llm = LLM(config=CFG, **KW)
    llm.args.return_all_prompt_logprobs = True
    llm.backend.args.return_all_prompt_logprobs = True
    prompt = np.random.default_rng(5).integers(3, 300, 70).tolist()
    req = llm._new_req(prompt, {"max_new_tokens": 2, "ignore_eos": True, "prompt_logprobs": 0,
                                "disable_prompt_cache": True})
    llm.queue.extend([req])
    from lightllm_b200.server.router.req_queue import Batch

    running = Batch(0, [])
    for _ in range(20):
        nb = llm.queue.generate_new_batch(running)
        if nb is not None:
            llm.backend.add_reqs(nb.reqs)
            running.merge(nb)
        if not llm.backend.has_work():
            break
        llm.backend.step()
        running.filter_out_finished_req()
    got = torch.tensor(req.shm_logprobs.arr[1:70])
    # the same numbers from one plain forward pass over the prompt
    m = LLM(config=CFG, **KW).model
    r = m.req_manager.alloc()
    ids = torch.tensor(prompt)
    mi = ModelInput(batch_size=1, total_token_num=70, max_kv_len=70, is_prefill=True,
                    b_req_idx=torch.tensor([r], dtype=torch.int32), b_seq_len=torch.tensor([70], dtype=torch.int32),
                    mem_indexes=m.mem_manager.alloc(70).clone(), input_ids=ids,
                    b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=70, return_all_logits=True)
    logp = torch.log_softmax(m.forward(mi).logits.float(), dim=-1)
    want = logp[torch.arange(69), ids[1:]]
    assert torch.allclose(got, want, atol=1e-4)


def test_outlines_index_regex_constraint():
    oc = pytest.importorskip("outlines_core")
    from lightllm_b200.engine.mode_backends import OutlinesConstraintBackend

    table = {}
    for i, t in enumerate(VOCAB):
        if i != 2:
            table.setdefault(t, []).append(i)
    llm = LLM(config=CFG, **KW)
    llm.backend = OutlinesConstraintBackend(llm.model, llm.args, vocabulary=oc.Vocabulary(2, table), is_master_in_dp=True)
    import re

    pat = r"(yes|no), [a-c]{3}\\."
    outs = llm.generate([[5, 6, 7], [9, 10, 11, 12], [20]], [{"max_new_tokens": 30, "regular_constraint": pat},
                                                            {"max_new_tokens": 30, "regular_constraint": pat},
                                                            {"max_new_tokens": 5, "ignore_eos": True}])
    for o in outs[:2]:
        assert re.fullmatch(pat, _text(o["token_ids"])) and o["finish_reason"] == "stop"
    assert len(outs[2]["token_ids"]) == 5
    assert len(llm.backend._indexes) == 1                       # the index of a pattern is built once


def test_backend_selection_from_start_arguments():
    from types import SimpleNamespace

    from lightllm_b200.engine import mode_backends as mb
    from lightllm_b200.engine.backend import ModelBackend

    def pick(**kw):
        return mb.select_backend_class(SimpleNamespace(**kw))

    assert pick() is ModelBackend
    assert pick(run_mode="prefill") is mb.PDPrefillBackend and pick(run_mode="decode") is mb.PDDecodeBackend
    assert pick(use_reward_model=True) is mb.RewardModelBackend
    assert pick(token_healing_mode=True) is mb.TokenHealingBackend
    assert pick(output_constraint_mode="xgrammar") is mb.XgrammarBackend
    assert pick(output_constraint_mode="outlines") in (mb.OutlinesConstraintBackend, mb.XgrammarBackend)
    assert pick(first_token_constraint_mode=True) is mb.FirstTokenConstraintBackend
    assert pick(diverse_mode=True) is mb.DiverseBackend
