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


QCFG = dict(model_type="qwen3_5_text", hidden_size=64, intermediate_size=128, num_hidden_layers=4,
            num_attention_heads=4, num_key_value_heads=2, head_dim=32, vocab_size=300, rms_norm_eps=1e-6,
            linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=16, linear_value_head_dim=16,
            linear_conv_kernel_dim=4, full_attention_interval=4, max_position_embeddings=512, eos_token_id=2,
            tie_word_embeddings=False)


@pytest.mark.parametrize("k", [1, 3])
def test_hybrid_target_rolls_its_recurrent_state_back(k):
    """Qwen3.5 (Gated DeltaNet layers) as the target: the linear layers' state after a verification pass is the
    state at the last accepted position, so speculative decoding still reproduces plain greedy decoding."""
    sp = {"max_new_tokens": 15, "ignore_eos": True}
    want = [o["token_ids"] for o in LLM(config=QCFG, **KW).generate(_prompts(), sp)]
    llm = LLM(config=QCFG, extra_kv_layers=1, **KW)
    drafts = build_mtp_modules(llm.model, 1)
    d = drafts[0]
    assert type(d).__name__ == "Qwen3_5MTP" and d.layer_types == ["full_attention"]
    assert d.kv_layer_offset == len(llm.model.full_layers)       # its KV layer follows the target's
    llm.backend = MTPBackend(llm.model, llm.args, draft_models=drafts, mtp_step=k, is_master_in_dp=True)
    got = llm.generate(_prompts(), sp)
    assert [o["token_ids"] for o in got] == want
    st = llm.backend.stats
    assert st["mtp_steps"] > 0 and st["mtp_accepted"] < st["mtp_proposed"]   # some drafts were rejected


def test_qwen3_5_draft_module_reads_the_mtp_prefix(tmp_path):
    """A checkpoint keeps the Qwen3.5 draft module under `mtp.`; the loader finds every tensor there."""
    from safetensors.torch import save_file

    llm = LLM(config=QCFG, extra_kv_layers=1, **KW)
    d0 = build_mtp_modules(llm.model, 1)[0]
    g = torch.Generator().manual_seed(5)
    ckpt = {}
    for name, shape in d0.weight_shapes().items():
        t = torch.randn(*shape, generator=g) * 0.05
        if name.startswith("model.layers.0."):
            rest = name[len("model.layers.0."):]
            new = {"eh_proj.weight": "mtp.fc.weight", "enorm.weight": "mtp.pre_fc_norm_embedding.weight",
                   "hnorm.weight": "mtp.pre_fc_norm_hidden.weight",
                   "shared_head.norm.weight": "mtp.norm.weight"}.get(rest, "mtp.layers.0." + rest)
        elif name == "model.norm.weight":
            continue
        else:
            new = {"model.embed_tokens.weight": "model.language_model.embed_tokens.weight"}.get(name, name)
        ckpt[new] = t
    save_file({k: v.contiguous() for k, v in ckpt.items()}, str(tmp_path / "model.safetensors"))
    d = build_mtp_modules(llm.model, 1, model_dir=str(tmp_path))[0]
    assert torch.equal(d.eh_proj_w.float(), ckpt["mtp.fc.weight"])
    assert torch.equal(d.final_norm_w.float(), ckpt["mtp.norm.weight"])
    assert torch.equal(d.layers[0].o_w.float(), ckpt["mtp.layers.0.self_attn.o_proj.weight"])
    assert d.embed_w is llm.model.embed_w                          # the big tables are the target's


def test_qwen3_5_moe_draft_module():
    cfg = dict(QCFG, model_type="qwen3_5_moe_text", num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
               shared_expert_intermediate_size=32, norm_topk_prob=True)
    sp = {"max_new_tokens": 9, "ignore_eos": True}
    want = [o["token_ids"] for o in LLM(config=cfg, **KW).generate(_prompts()[:2], sp)]
    llm = LLM(config=cfg, extra_kv_layers=1, **KW)
    drafts = build_mtp_modules(llm.model, 1)
    assert type(drafts[0]).__name__ == "Qwen3_5MoeMTP" and drafts[0].moe is not None
    llm.backend = MTPBackend(llm.model, llm.args, draft_models=drafts, mtp_step=2, is_master_in_dp=True)
    assert [o["token_ids"] for o in llm.generate(_prompts()[:2], sp)] == want
