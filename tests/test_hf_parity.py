"""Logit parity with the Hugging Face implementations on CPU: a tiny random-weight checkpoint of each family is
saved by transformers and loaded by this package (safetensors path, fp32), then prefill logits of one prompt and
a decode step are compared."""
import os

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _run_ours(model_dir, ids, extra_steps=2):
    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.base import load_config
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.parallel import dist as pdist

    ps = pdist.ParallelState(device=torch.device("cpu"))
    m = get_model(load_config(model_dir), model_dir=model_dir, pstate=ps, data_type="float32", max_total_token_num=512,
                  max_req_num=4, max_seq_length=256, disable_cudagraph=True)
    req = m.req_manager.alloc()
    n = len(ids)
    slots = m.mem_manager.alloc(n)
    mi = ModelInput(batch_size=1, total_token_num=n, max_kv_len=n, is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([n], dtype=torch.int32),
                    mem_indexes=slots.clone(), input_ids=ids.clone(), b_ready_cache_len=torch.zeros(1, dtype=torch.int32),
                    max_q_len=n, return_all_logits=True)
    out = [m.forward(mi).logits.float()]
    seq = ids.tolist()
    for _ in range(extra_steps):  # greedy decode steps through the decode path
        nxt = int(out[-1][-1].argmax())
        seq.append(nxt)
        m.req_manager.req_to_next_token_ids[req] = nxt
        slot = m.mem_manager.alloc(1)
        mi = ModelInput(batch_size=1, total_token_num=len(seq), max_kv_len=len(seq), is_prefill=False,
                        b_req_idx=torch.tensor([req], dtype=torch.int32),
                        b_seq_len=torch.tensor([len(seq)], dtype=torch.int32), mem_indexes=slot.clone())
        out.append(m.forward(mi).logits.float())
    return out, seq


def _check(tmp_path, hf_model, ids, tol=2e-3):
    d = str(tmp_path / "ckpt")
    hf_model = hf_model.eval().float()
    hf_model.save_pretrained(d, safe_serialization=True)
    ours, seq = _run_ours(d, ids)
    with torch.no_grad():
        ref = hf_model(torch.tensor([seq])).logits[0].float()
    n = len(ids)
    scale = ref.abs().max().item()
    err = (ours[0] - ref[:n]).abs().max().item()
    assert err < tol * max(scale, 1.0), f"prefill logits differ: {err} (scale {scale})"
    for k, o in enumerate(ours[1:]):
        err = (o[0] - ref[n + k]).abs().max().item()
        assert err < tol * max(scale, 1.0), f"decode step {k} logits differ: {err} (scale {scale})"


def _ids(vocab, n=23, seed=0):
    return torch.randint(3, vocab, (n,), generator=torch.Generator().manual_seed(seed))


def test_llama(tmp_path):
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=200, max_position_embeddings=256, rope_theta=10000.0)
    _check(tmp_path, LlamaForCausalLM(cfg), _ids(200))


def test_qwen2(tmp_path):
    from transformers import Qwen2Config, Qwen2ForCausalLM

    torch.manual_seed(0)
    cfg = Qwen2Config(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=200, max_position_embeddings=256)
    _check(tmp_path, Qwen2ForCausalLM(cfg), _ids(200))


def test_qwen3(tmp_path):
    from transformers import Qwen3Config, Qwen3ForCausalLM

    torch.manual_seed(0)
    cfg = Qwen3Config(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=32, vocab_size=200, max_position_embeddings=256)
    _check(tmp_path, Qwen3ForCausalLM(cfg), _ids(200))


def test_mistral(tmp_path):
    from transformers import MistralConfig, MistralForCausalLM

    torch.manual_seed(0)
    cfg = MistralConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, vocab_size=200, max_position_embeddings=256, sliding_window=None)
    _check(tmp_path, MistralForCausalLM(cfg), _ids(200))


def test_qwen3_moe(tmp_path):
    from transformers import Qwen3MoeConfig, Qwen3MoeForCausalLM

    torch.manual_seed(0)
    cfg = Qwen3MoeConfig(hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=32, num_experts=8, num_experts_per_tok=2,
                         norm_topk_prob=True, vocab_size=200, max_position_embeddings=256, decoder_sparse_step=1,
                         mlp_only_layers=[])
    _check(tmp_path, Qwen3MoeForCausalLM(cfg), _ids(200))


def test_mixtral(tmp_path):
    from transformers import MixtralConfig, MixtralForCausalLM

    torch.manual_seed(0)
    cfg = MixtralConfig(hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, num_local_experts=4, num_experts_per_tok=2, vocab_size=200,
                        max_position_embeddings=256, sliding_window=None)
    _check(tmp_path, MixtralForCausalLM(cfg), _ids(200))


def test_deepseek_v3(tmp_path):
    from transformers import DeepseekV3Config, DeepseekV3ForCausalLM

    torch.manual_seed(0)
    cfg = DeepseekV3Config(hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=3,
                           num_attention_heads=4, num_key_value_heads=4, n_routed_experts=8, n_shared_experts=1,
                           num_experts_per_tok=2, n_group=2, topk_group=1, first_k_dense_replace=1, q_lora_rank=32,
                           kv_lora_rank=48, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, vocab_size=200,
                           max_position_embeddings=256, routed_scaling_factor=2.5, norm_topk_prob=True,
                           rope_scaling=None)
    m = DeepseekV3ForCausalLM(cfg)
    with torch.no_grad():  # a non-trivial routing bias
        for layer in m.model.layers[1:]:
            layer.mlp.gate.e_score_correction_bias.copy_(torch.randn(8) * 0.1)
    _check(tmp_path, m, _ids(200))
