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


def test_bloom(tmp_path):
    from transformers import BloomConfig, BloomForCausalLM

    torch.manual_seed(0)
    cfg = BloomConfig(hidden_size=64, n_layer=2, n_head=4, vocab_size=200)
    _check(tmp_path, BloomForCausalLM(cfg), _ids(200))


def test_gpt_bigcode(tmp_path):
    from transformers import GPTBigCodeConfig, GPTBigCodeForCausalLM

    torch.manual_seed(0)
    cfg = GPTBigCodeConfig(n_embd=64, n_layer=2, n_head=4, n_inner=128, vocab_size=200, n_positions=256,
                           multi_query=True)
    _check(tmp_path, GPTBigCodeForCausalLM(cfg), _ids(200))


def test_starcoder2(tmp_path):
    from transformers import Starcoder2Config, Starcoder2ForCausalLM

    torch.manual_seed(0)
    cfg = Starcoder2Config(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                           num_key_value_heads=2, vocab_size=200, max_position_embeddings=256, sliding_window=16)
    _check(tmp_path, Starcoder2ForCausalLM(cfg), _ids(200, n=40))


def test_stablelm(tmp_path):
    from transformers import StableLmConfig, StableLmForCausalLM

    torch.manual_seed(0)
    cfg = StableLmConfig(hidden_size=96, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=4, vocab_size=200, max_position_embeddings=256, partial_rotary_factor=0.25,
                         use_qkv_bias=True)
    _check(tmp_path, StableLmForCausalLM(cfg), _ids(200))


def test_phi3(tmp_path):
    from transformers import Phi3Config, Phi3ForCausalLM

    torch.manual_seed(0)
    cfg = Phi3Config(hidden_size=96, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, vocab_size=200, max_position_embeddings=256, pad_token_id=0)
    _check(tmp_path, Phi3ForCausalLM(cfg), _ids(200))


def test_gemma(tmp_path):
    from transformers import GemmaConfig, GemmaForCausalLM

    torch.manual_seed(0)
    cfg = GemmaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=1, head_dim=32, vocab_size=200, max_position_embeddings=256)
    _check(tmp_path, GemmaForCausalLM(cfg), _ids(200))


def test_gemma3_text(tmp_path):
    from transformers import Gemma3ForCausalLM, Gemma3TextConfig

    torch.manual_seed(0)
    cfg = Gemma3TextConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=6, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=32, vocab_size=200, max_position_embeddings=256,
                           sliding_window=8, query_pre_attn_scalar=32)
    _check(tmp_path, Gemma3ForCausalLM(cfg), _ids(200, n=30))


# ---- families without a transformers class: the same math under another checkpoint layout ----
def _save_custom(tmp_path, cfg: dict, tensors: dict):
    import json

    from safetensors.torch import save_file

    d = tmp_path / "custom"
    d.mkdir()
    with open(d / "config.json", "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(d / "model.safetensors"))
    return str(d)


def _compare(model_dir, hf_model, ids, tol=2e-3):
    ours, seq = _run_ours(model_dir, ids)
    with torch.no_grad():
        ref = hf_model(torch.tensor([seq])).logits[0].float()
    n = len(ids)
    assert (ours[0] - ref[:n]).abs().max().item() < tol * max(ref.abs().max().item(), 1.0)
    for k, o in enumerate(ours[1:]):
        assert (o[0] - ref[n + k]).abs().max().item() < tol * max(ref.abs().max().item(), 1.0)


def test_internlm2_layout(tmp_path):
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    H, nh, nkv, L = 64, 4, 2, 2
    D, g = H // nh, nh // nkv
    hf = LlamaForCausalLM(LlamaConfig(hidden_size=H, intermediate_size=128, num_hidden_layers=L, num_attention_heads=nh,
                                      num_key_value_heads=nkv, vocab_size=200, max_position_embeddings=256)).eval().float()
    sd = hf.state_dict()
    t = {"model.tok_embeddings.weight": sd["model.embed_tokens.weight"], "model.norm.weight": sd["model.norm.weight"],
         "output.weight": sd["lm_head.weight"]}
    for i in range(L):
        p = f"model.layers.{i}."
        q = sd[p + "self_attn.q_proj.weight"].view(nkv, g, D, H)
        k = sd[p + "self_attn.k_proj.weight"].view(nkv, 1, D, H)
        v = sd[p + "self_attn.v_proj.weight"].view(nkv, 1, D, H)
        t[p + "attention.wqkv.weight"] = torch.cat([q, k, v], dim=1).reshape(-1, H)
        t[p + "attention.wo.weight"] = sd[p + "self_attn.o_proj.weight"]
        t[p + "feed_forward.w1.weight"] = sd[p + "mlp.gate_proj.weight"]
        t[p + "feed_forward.w3.weight"] = sd[p + "mlp.up_proj.weight"]
        t[p + "feed_forward.w2.weight"] = sd[p + "mlp.down_proj.weight"]
        t[p + "attention_norm.weight"] = sd[p + "input_layernorm.weight"]
        t[p + "ffn_norm.weight"] = sd[p + "post_attention_layernorm.weight"]
    cfg = dict(model_type="internlm2", hidden_size=H, intermediate_size=128, num_hidden_layers=L, num_attention_heads=nh,
               num_key_value_heads=nkv, vocab_size=200, rms_norm_eps=hf.config.rms_norm_eps, rope_theta=10000.0)
    _compare(_save_custom(tmp_path, cfg, t), hf, _ids(200))


def test_qwen_v1_layout(tmp_path):
    from transformers import Qwen2Config, Qwen2ForCausalLM

    torch.manual_seed(0)
    H, nh, L, I = 64, 4, 2, 96
    hf = Qwen2ForCausalLM(Qwen2Config(hidden_size=H, intermediate_size=I, num_hidden_layers=L, num_attention_heads=nh,
                                      num_key_value_heads=nh, vocab_size=200, max_position_embeddings=256,
                                      tie_word_embeddings=False)).eval().float()
    sd = hf.state_dict()
    t = {"transformer.wte.weight": sd["model.embed_tokens.weight"], "transformer.ln_f.weight": sd["model.norm.weight"],
         "lm_head.weight": sd["lm_head.weight"]}
    for i in range(L):
        p, q = f"model.layers.{i}.", f"transformer.h.{i}."
        t[q + "attn.c_attn.weight"] = torch.cat([sd[p + f"self_attn.{n}_proj.weight"] for n in "qkv"], dim=0)
        t[q + "attn.c_attn.bias"] = torch.cat([sd[p + f"self_attn.{n}_proj.bias"] for n in "qkv"], dim=0)
        t[q + "attn.c_proj.weight"] = sd[p + "self_attn.o_proj.weight"]
        t[q + "mlp.w2.weight"] = sd[p + "mlp.gate_proj.weight"]
        t[q + "mlp.w1.weight"] = sd[p + "mlp.up_proj.weight"]
        t[q + "mlp.c_proj.weight"] = sd[p + "mlp.down_proj.weight"]
        t[q + "ln_1.weight"] = sd[p + "input_layernorm.weight"]
        t[q + "ln_2.weight"] = sd[p + "post_attention_layernorm.weight"]
    cfg = dict(model_type="qwen", hidden_size=H, intermediate_size=2 * I, num_hidden_layers=L, num_attention_heads=nh,
               vocab_size=200, layer_norm_epsilon=hf.config.rms_norm_eps, rotary_emb_base=10000.0)
    _compare(_save_custom(tmp_path, cfg, t), hf, _ids(200))


def test_minicpm_scales(tmp_path):
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    H, L = 64, 2
    s_e, depth, base = 12.0, 1.4, 32
    hf = LlamaForCausalLM(LlamaConfig(hidden_size=H, intermediate_size=128, num_hidden_layers=L, num_attention_heads=4,
                                      num_key_value_heads=2, vocab_size=200, max_position_embeddings=256,
                                      tie_word_embeddings=False)).eval().float()
    raw = {k: v.clone() for k, v in hf.state_dict().items()}  # the MiniCPM checkpoint: unscaled tensors
    with torch.no_grad():  # the reference: the same network with the scales folded into the weights
        hf.model.embed_tokens.weight.mul_(s_e)
        hf.lm_head.weight.mul_(1.0 / (H / base))
        for layer in hf.model.layers:
            layer.self_attn.o_proj.weight.mul_(depth / L ** 0.5)
            layer.mlp.down_proj.weight.mul_(depth / L ** 0.5)
    cfg = dict(model_type="minicpm", hidden_size=H, intermediate_size=128, num_hidden_layers=L, num_attention_heads=4,
               num_key_value_heads=2, vocab_size=200, rms_norm_eps=hf.config.rms_norm_eps, rope_theta=10000.0,
               scale_emb=s_e, scale_depth=depth, dim_model_base=base, tie_word_embeddings=False)
    _compare(_save_custom(tmp_path, cfg, raw), hf, _ids(200))


def test_internlm_bias(tmp_path):
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    hf = LlamaForCausalLM(LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                      num_key_value_heads=4, vocab_size=200, max_position_embeddings=256,
                                      attention_bias=True)).eval().float()
    with torch.no_grad():
        for layer in hf.model.layers:
            for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
                getattr(layer.self_attn, n).bias.normal_(0, 0.1)
    cfg = dict(model_type="internlm", hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               vocab_size=200, rms_norm_eps=hf.config.rms_norm_eps, rope_theta=10000.0, bias=True)
    _compare(_save_custom(tmp_path, cfg, dict(hf.state_dict())), hf, _ids(200))


def test_qwen2_vl_vision_tower_mrope_and_merge(tmp_path):
    """Pixels -> vision tower -> embedding arena -> M-RoPE language model, against Qwen2VLForConditionalGeneration."""
    from transformers import Qwen2VLConfig, Qwen2VLForConditionalGeneration

    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.base import load_config
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.models.vit.qwen2_vl_visual import Qwen2VLVisionTower, patchify
    from lightllm_b200.models.weights import SafetensorsSource
    from lightllm_b200.parallel import dist as pdist

    torch.manual_seed(0)
    text = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                vocab_size=300, max_position_embeddings=512, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]})
    vision = dict(depth=2, embed_dim=32, hidden_size=64, num_heads=4, mlp_ratio=2, patch_size=14, spatial_merge_size=2,
                  temporal_patch_size=2, in_chans=3)
    cfg = Qwen2VLConfig(text_config=text, vision_config=vision, image_token_id=290, video_token_id=291,
                        vision_start_token_id=292, vision_end_token_id=293)
    hf = Qwen2VLForConditionalGeneration(cfg).eval().float()
    d = str(tmp_path / "ckpt")
    hf.save_pretrained(d, safe_serialization=True)

    # one 56 x 84 image: 4 x 6 patches -> 2 x 3 = 6 merged tokens
    pixels = torch.randn(1, 3, 56, 84)
    patches, (t, gh, gw) = patchify(pixels)
    n_img = t * gh * gw // 4
    assert n_img == 6
    pre, post = [5, 17, 292], [293, 9, 44, 120, 7]
    hf_ids = torch.tensor([pre + [290] * n_img + post])
    with torch.no_grad():
        ref = hf(input_ids=hf_ids, pixel_values=patches, image_grid_thw=torch.tensor([[t, gh, gw]]),
                 mm_token_type_ids=(hf_ids == 290).long()).logits[0].float()

    src = SafetensorsSource(d)
    tower = Qwen2VLVisionTower(load_config(d)["vision_config"], src, torch.device("cpu"), torch.float32)
    emb = tower.forward(patches, [(t, gh, gw)])
    with torch.no_grad():
        want = hf.model.visual(patches, grid_thw=torch.tensor([[t, gh, gw]]))
        want = want.pooler_output if hasattr(want, "pooler_output") else want
    assert (emb - want).abs().max().item() < 1e-4

    class Arena:  # stand-in for the shared embedding arena
        def read_rows(self, rows):
            return emb[rows - 40]

    ps = pdist.ParallelState(device=torch.device("cpu"))
    m = get_model(load_config(d), model_dir=d, pstate=ps, data_type="float32", max_total_token_num=256, max_req_num=2,
                  max_seq_length=128, disable_cudagraph=True)
    m.embed_arena = Arena()
    tok0 = 100_000_000
    ids = torch.tensor(pre + list(range(tok0, tok0 + n_img)) + post)
    item = {"token_id": tok0, "token_num": n_img, "start_index_in_embed_cache": 40, "grid_thwd": (t, gh, gw, 2)}
    req, n = m.req_manager.alloc(), len(ids)
    slots = m.mem_manager.alloc(n)
    mi = ModelInput(batch_size=1, total_token_num=n, max_kv_len=n, is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([n], dtype=torch.int32),
                    mem_indexes=slots.clone(), input_ids=ids, b_ready_cache_len=torch.zeros(1, dtype=torch.int32),
                    max_q_len=n, return_all_logits=True, multimodal_params=[{"images": [item], "audios": []}])
    got = m.forward(mi).logits.float()
    assert (got - ref).abs().max().item() < 2e-3 * max(ref.abs().max().item(), 1.0)
    # one decode step: the position continues after the image's largest index
    nxt = int(ref[-1].argmax())
    with torch.no_grad():
        ids2 = torch.cat([hf_ids, torch.tensor([[nxt]])], dim=1)
        ref2 = hf(input_ids=ids2, pixel_values=patches, image_grid_thw=torch.tensor([[t, gh, gw]]),
                  mm_token_type_ids=(ids2 == 290).long()).logits[0, -1].float()
    m.req_manager.req_to_next_token_ids[req] = nxt
    mi = ModelInput(batch_size=1, total_token_num=n + 1, max_kv_len=n + 1, is_prefill=False,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([n + 1], dtype=torch.int32),
                    mem_indexes=m.mem_manager.alloc(1).clone())
    got2 = m.forward(mi).logits.float()[0]
    assert (got2 - ref2).abs().max().item() < 2e-3 * max(ref.abs().max().item(), 1.0)


def test_gpt_oss(tmp_path):
    from transformers import GptOssConfig, GptOssForCausalLM

    torch.manual_seed(0)
    cfg = GptOssConfig(hidden_size=64, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=16, num_local_experts=4, num_experts_per_tok=2, vocab_size=200,
                       max_position_embeddings=256, sliding_window=8, rope_scaling=None,
                       layer_types=["sliding_attention", "full_attention"])
    m = GptOssForCausalLM(cfg)
    with torch.no_grad():
        for layer in m.model.layers:
            layer.self_attn.sinks.normal_(0, 1)
            layer.mlp.router.bias.normal_(0, 0.5)
            layer.mlp.experts.gate_up_proj_bias.normal_(0, 0.5)
            layer.mlp.experts.down_proj_bias.normal_(0, 0.5)
            layer.mlp.experts.gate_up_proj.normal_(0, 0.3)
            layer.mlp.experts.down_proj.normal_(0, 0.3)
    _check(tmp_path, m, _ids(200, n=30))


def test_llava_clip_tower_and_merge(tmp_path):
    from transformers import CLIPVisionConfig, LlamaConfig, LlavaConfig, LlavaForConditionalGeneration

    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.base import load_config
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.models.vit.clip_visual import ClipLlavaTower
    from lightllm_b200.models.weights import SafetensorsSource
    from lightllm_b200.parallel import dist as pdist
    import json
    import os

    torch.manual_seed(0)
    vc = CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                          image_size=28, patch_size=14)
    tc = LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, vocab_size=300, max_position_embeddings=256)
    cfg = LlavaConfig(vision_config=vc, text_config=tc, image_token_index=290)
    hf = LlavaForConditionalGeneration(cfg).eval().float()
    d = str(tmp_path / "ckpt")
    hf.save_pretrained(d, safe_serialization=True)
    pixels = torch.randn(1, 3, 28, 28)
    n_img = 4
    pre, post = [5, 17], [9, 44, 120]
    hf_ids = torch.tensor([pre + [290] * n_img + post])
    with torch.no_grad():
        ref = hf(input_ids=hf_ids, pixel_values=pixels).logits[0].float()
    raw_cfg = json.load(open(os.path.join(d, "config.json")))
    tower = ClipLlavaTower(raw_cfg, SafetensorsSource(d), torch.device("cpu"), torch.float32)
    emb = tower.forward(pixels)[0]
    assert emb.shape == (n_img, 64) and tower.tokens_per_image == n_img

    class Arena:
        def read_rows(self, rows):
            return emb[rows - 7]

    ps = pdist.ParallelState(device=torch.device("cpu"))
    m = get_model(load_config(d), model_dir=d, pstate=ps, data_type="float32", max_total_token_num=256, max_req_num=2,
                  max_seq_length=128, disable_cudagraph=True)
    m.embed_arena = Arena()
    tok0 = 100_000_000
    ids = torch.tensor(pre + list(range(tok0, tok0 + n_img)) + post)
    item = {"token_id": tok0, "token_num": n_img, "start_index_in_embed_cache": 7}
    req, n = m.req_manager.alloc(), len(ids)
    mi = ModelInput(batch_size=1, total_token_num=n, max_kv_len=n, is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([n], dtype=torch.int32),
                    mem_indexes=m.mem_manager.alloc(n).clone(), input_ids=ids,
                    b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=n, return_all_logits=True,
                    multimodal_params=[{"images": [item], "audios": []}])
    got = m.forward(mi).logits.float()
    assert (got - ref).abs().max().item() < 2e-3 * max(ref.abs().max().item(), 1.0)


def test_qwen3_vl_tower_deepstack_and_interleaved_mrope(tmp_path):
    """Pixels -> Qwen3-VL tower (interpolated position table, deep-stack mergers) -> arena rows [embedding | deep-stack
    sets] -> Qwen3 decoder with interleaved M-RoPE and deep-stack adds, against Qwen3VLForConditionalGeneration."""
    from transformers import Qwen3VLConfig, Qwen3VLForConditionalGeneration

    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.base import embed_row_width, load_config
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.models.vit.qwen2_vl_visual import patchify
    from lightllm_b200.models.vit.qwen3_vl_visual import Qwen3VLVisionTower
    from lightllm_b200.models.weights import SafetensorsSource
    from lightllm_b200.parallel import dist as pdist

    torch.manual_seed(0)
    text = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                head_dim=16, vocab_size=300, max_position_embeddings=512,
                rope_scaling={"rope_type": "default", "mrope_section": [2, 3, 3], "mrope_interleaved": True})
    vision = dict(depth=3, hidden_size=32, num_heads=4, intermediate_size=64, out_hidden_size=64, patch_size=16,
                  spatial_merge_size=2, temporal_patch_size=2, in_channels=3, num_position_embeddings=36,
                  deepstack_visual_indexes=[0, 2], hidden_act="gelu_pytorch_tanh")
    cfg = Qwen3VLConfig(text_config=text, vision_config=vision, image_token_id=290, video_token_id=291,
                        vision_start_token_id=292, vision_end_token_id=293, tie_word_embeddings=False)
    hf = Qwen3VLForConditionalGeneration(cfg).eval().float()
    d = str(tmp_path / "ckpt")
    hf.save_pretrained(d, safe_serialization=True)

    pixels = torch.randn(1, 3, 64, 96)   # 4 x 6 patches -> 2 x 3 = 6 merged tokens
    patches, (t, gh, gw) = patchify(pixels, patch=16)
    n_img = t * gh * gw // 4
    assert n_img == 6
    pre, post = [5, 17, 292], [293, 9, 44, 120, 7]
    hf_ids = torch.tensor([pre + [290] * n_img + post])
    with torch.no_grad():
        ref = hf(input_ids=hf_ids, pixel_values=patches, image_grid_thw=torch.tensor([[t, gh, gw]]),
                 mm_token_type_ids=(hf_ids == 290).long()).logits[0].float()
        vis = hf.model.visual(patches, grid_thw=torch.tensor([[t, gh, gw]]))

    conf = load_config(d)
    assert embed_row_width(conf) == 64 * 3
    src = SafetensorsSource(d)
    tower = Qwen3VLVisionTower(conf["vision_config"], src, torch.device("cpu"), torch.float32)
    emb = tower.forward(patches, [(t, gh, gw)])
    assert emb.shape == (n_img, 64 * 3)
    assert (emb[:, :64] - vis.pooler_output).abs().max().item() < 1e-4
    for j, f in enumerate(vis.deepstack_features):
        assert (emb[:, 64 * (j + 1):64 * (j + 2)] - f).abs().max().item() < 1e-4
    assert set(Qwen3VLVisionTower.weight_shapes(conf["vision_config"])) <= set(src.names())

    class Arena:
        def read_rows(self, rows):
            return emb[rows - 40]

    ps = pdist.ParallelState(device=torch.device("cpu"))
    m = get_model(conf, model_dir=d, pstate=ps, data_type="float32", max_total_token_num=256, max_req_num=2,
                  max_seq_length=128, disable_cudagraph=True)
    assert type(m).__name__ == "Qwen3VLLM" and m.embed_row_width == 192
    m.embed_arena = Arena()
    tok0 = 100_000_000
    ids = torch.tensor(pre + list(range(tok0, tok0 + n_img)) + post)
    item = {"token_id": tok0, "token_num": n_img, "start_index_in_embed_cache": 40, "grid_thwd": (t, gh, gw, 2)}
    req, n = m.req_manager.alloc(), len(ids)
    mi = ModelInput(batch_size=1, total_token_num=n, max_kv_len=n, is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([n], dtype=torch.int32),
                    mem_indexes=m.mem_manager.alloc(n).clone(), input_ids=ids,
                    b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=n, return_all_logits=True,
                    multimodal_params=[{"images": [item], "audios": []}])
    got = m.forward(mi).logits.float()
    assert (got - ref).abs().max().item() < 2e-3 * max(ref.abs().max().item(), 1.0)


def test_qwen3_vl_moe_fused_expert_tensors(tmp_path):
    """Qwen3-VL-MoE text path (no image): experts stored as 3-D tensors are split per expert at load."""
    from transformers import Qwen3VLMoeConfig, Qwen3VLMoeForConditionalGeneration

    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.base import load_config
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.parallel import dist as pdist

    torch.manual_seed(0)
    text = dict(hidden_size=64, intermediate_size=128, moe_intermediate_size=64, num_experts=4, num_experts_per_tok=2,
                num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=300,
                decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True, max_position_embeddings=256,
                rope_scaling={"rope_type": "default", "mrope_section": [2, 3, 3], "mrope_interleaved": True})
    vision = dict(depth=1, hidden_size=32, num_heads=4, intermediate_size=64, out_hidden_size=64, patch_size=16,
                  spatial_merge_size=2, temporal_patch_size=2, in_channels=3, num_position_embeddings=36,
                  deepstack_visual_indexes=[0])
    cfg = Qwen3VLMoeConfig(text_config=text, vision_config=vision, image_token_id=290, tie_word_embeddings=False)
    hf = Qwen3VLMoeForConditionalGeneration(cfg).eval().float()
    d = str(tmp_path / "ckpt")
    hf.save_pretrained(d, safe_serialization=True)
    ids = torch.randint(3, 280, (23,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = hf(input_ids=ids.unsqueeze(0)).logits[0].float()
    m = get_model(load_config(d), model_dir=d, pstate=pdist.ParallelState(device=torch.device("cpu")),
                  data_type="float32", max_total_token_num=128, max_req_num=2, max_seq_length=64, disable_cudagraph=True)
    assert type(m).__name__ == "Qwen3VLMoeLM" and m.layers[0].w13.shape == (4, 128, 64)
    req, n = m.req_manager.alloc(), len(ids)
    mi = ModelInput(batch_size=1, total_token_num=n, max_kv_len=n, is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([n], dtype=torch.int32),
                    mem_indexes=m.mem_manager.alloc(n).clone(), input_ids=ids,
                    b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=n, return_all_logits=True)
    got = m.forward(mi).logits.float()
    assert (got - ref).abs().max().item() < 2e-3 * max(ref.abs().max().item(), 1.0)


def test_qwen3_next_hybrid_linear_attention(tmp_path):
    """Qwen3-Next: Gated DeltaNet layers (convolution + matrix state carried over chunks and decode steps), gated
    softmax attention with partial rotary embedding, shared expert with a sigmoid gate, against Hugging Face."""
    from transformers import Qwen3NextConfig, Qwen3NextForCausalLM

    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.base import load_config
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.parallel import dist as pdist

    torch.manual_seed(0)
    cfg = Qwen3NextConfig(hidden_size=64, intermediate_size=128, moe_intermediate_size=32,
                          shared_expert_intermediate_size=32, num_experts=4, num_experts_per_tok=2,
                          num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                          vocab_size=300, linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=16,
                          linear_value_head_dim=16, linear_conv_kernel_dim=4, full_attention_interval=4,
                          partial_rotary_factor=0.25, decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True,
                          max_position_embeddings=256, tie_word_embeddings=False)
    hf = Qwen3NextForCausalLM(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n or "dt_bias" in n or "A_log" in n:
                p.add_(torch.randn_like(p) * 0.1)
    d = str(tmp_path / "ckpt")
    hf.save_pretrained(d, safe_serialization=True)
    ids = torch.randint(3, 280, (90,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = hf(input_ids=ids.unsqueeze(0)).logits[0].float()

    m = get_model(load_config(d), model_dir=d, pstate=pdist.ParallelState(device=torch.device("cpu")),
                  data_type="float32", max_total_token_num=256, max_req_num=3, max_seq_length=128, disable_cudagraph=True)
    assert m.full_layers == [3] and m.mem_manager.layer(0) is not None and not m.supports_prefix_cache
    scale = max(ref.abs().max().item(), 1.0)

    def prefill(req, tokens, ready):
        n = len(tokens)
        mi = ModelInput(batch_size=1, total_token_num=ready + n, max_kv_len=ready + n, is_prefill=True,
                        b_req_idx=torch.tensor([req], dtype=torch.int32),
                        b_seq_len=torch.tensor([ready + n], dtype=torch.int32),
                        mem_indexes=m.mem_manager.alloc(n).clone(), input_ids=tokens,
                        b_ready_cache_len=torch.tensor([ready], dtype=torch.int32), max_q_len=n, return_all_logits=True)
        return m.forward(mi).logits.float()

    # whole prompt of 70 tokens in one pass, then 20 decode steps fed with the reference tokens
    r0 = m.req_manager.alloc()
    got = prefill(r0, ids[:70], 0)
    assert (got - ref[:70]).abs().max().item() < 2e-3 * scale
    for t in range(70, 74):
        m.req_manager.req_to_next_token_ids[r0] = int(ids[t])
        mi = ModelInput(batch_size=1, total_token_num=t + 1, max_kv_len=t + 1, is_prefill=False,
                        b_req_idx=torch.tensor([r0], dtype=torch.int32),
                        b_seq_len=torch.tensor([t + 1], dtype=torch.int32), mem_indexes=m.mem_manager.alloc(1).clone())
        step = m.forward(mi).logits.float()
        assert (step[0] - ref[t]).abs().max().item() < 2e-3 * scale, f"decode step at position {t}"
    # chunked prefill of another request: 37 + 53 tokens, the state travels from the first chunk to the second
    r1 = m.req_manager.alloc()
    a = prefill(r1, ids[:37], 0)
    b = prefill(r1, ids[37:], 37)
    assert (torch.cat([a, b]) - ref).abs().max().item() < 2e-3 * scale


def test_qwen3_5_text_model_separate_projections(tmp_path):
    """Qwen3.5 dense text model: in_proj_qkv / z / b / a stored separately, regrouped per key head at load."""
    from transformers.models.qwen3_5 import modeling_qwen3_5 as hfm
    from transformers import Qwen3_5TextConfig

    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.base import load_config
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.parallel import dist as pdist

    torch.manual_seed(0)
    tc = Qwen3_5TextConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=32, vocab_size=300, linear_num_value_heads=4,
                           linear_num_key_heads=2, linear_key_head_dim=16, linear_value_head_dim=16,
                           linear_conv_kernel_dim=4, full_attention_interval=4, max_position_embeddings=256,
                           tie_word_embeddings=False)
    hf = hfm.Qwen3_5ForCausalLM(tc).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n or "dt_bias" in n or "A_log" in n:
                p.add_(torch.randn_like(p) * 0.1)
    d = str(tmp_path / "ckpt")
    hf.save_pretrained(d, safe_serialization=True)
    ids = torch.randint(3, 280, (50,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = hf(input_ids=ids.unsqueeze(0)).logits[0].float()
    m = get_model(load_config(d), model_dir=d, pstate=pdist.ParallelState(device=torch.device("cpu")),
                  data_type="float32", max_total_token_num=128, max_req_num=2, max_seq_length=64, disable_cudagraph=True)
    assert type(m).__name__ == "Qwen3_5LM"
    req, n = m.req_manager.alloc(), len(ids)
    mi = ModelInput(batch_size=1, total_token_num=n, max_kv_len=n, is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([n], dtype=torch.int32),
                    mem_indexes=m.mem_manager.alloc(n).clone(), input_ids=ids,
                    b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=n, return_all_logits=True)
    got = m.forward(mi).logits.float()
    assert (got - ref).abs().max().item() < 2e-3 * max(ref.abs().max().item(), 1.0)


def test_gemma3_siglip_tower_and_bidirectional_picture_tokens(tmp_path):
    from transformers import Gemma3Config, Gemma3ForConditionalGeneration

    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.base import load_config
    from lightllm_b200.models.registry import get_model, is_multimodal
    from lightllm_b200.models.vit.siglip_visual import SiglipGemma3Tower
    from lightllm_b200.models.weights import SafetensorsSource
    from lightllm_b200.parallel import dist as pdist
    import json
    import os

    torch.manual_seed(0)
    text = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=2, num_key_value_heads=1,
                head_dim=32, vocab_size=300, sliding_window=64, query_pre_attn_scalar=32, max_position_embeddings=256,
                layer_types=["sliding_attention", "sliding_attention", "full_attention"])
    vision = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=56,
                  patch_size=14, num_channels=3)
    cfg = Gemma3Config(text_config=text, vision_config=vision, mm_tokens_per_image=4, image_token_index=290,
                       boi_token_index=291, eoi_token_index=292)
    hf = Gemma3ForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        hf.model.multi_modal_projector.mm_input_projection_weight.normal_(0, 0.1)
    d = str(tmp_path / "ckpt")
    hf.save_pretrained(d, safe_serialization=True)
    pixels = torch.randn(1, 3, 56, 56)
    n_img = 4
    pre, post = [5, 17, 291], [292, 9, 44, 120]
    hf_ids = torch.tensor([pre + [290] * n_img + post])
    with torch.no_grad():
        ref = hf(input_ids=hf_ids, pixel_values=pixels, token_type_ids=(hf_ids == 290).long()).logits[0].float()
        feats = hf.model.get_image_features(pixels)
        want_emb = (feats.pooler_output if hasattr(feats, "pooler_output") else feats).reshape(n_img, -1)
    raw_cfg = json.load(open(os.path.join(d, "config.json")))
    assert is_multimodal(load_config(d))
    tower = SiglipGemma3Tower(raw_cfg, SafetensorsSource(d), torch.device("cpu"), torch.float32)
    emb = tower.forward(pixels)[0]
    assert (emb - want_emb).abs().max().item() < 1e-4

    class Arena:
        def read_rows(self, rows):
            return emb[rows - 3]

    m = get_model(load_config(d), model_dir=d, pstate=pdist.ParallelState(device=torch.device("cpu")),
                  data_type="float32", max_total_token_num=256, max_req_num=2, max_seq_length=128, disable_cudagraph=True)
    assert type(m).__name__ == "Gemma3LM"
    m.embed_arena = Arena()
    tok0 = 100_000_000
    ids = torch.tensor(pre + list(range(tok0, tok0 + n_img)) + post)
    item = {"token_id": tok0, "token_num": n_img, "start_index_in_embed_cache": 3}
    req, n = m.req_manager.alloc(), len(ids)
    mi = ModelInput(batch_size=1, total_token_num=n, max_kv_len=n, is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([n], dtype=torch.int32),
                    mem_indexes=m.mem_manager.alloc(n).clone(), input_ids=ids,
                    b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=n, return_all_logits=True,
                    multimodal_params=[{"images": [item], "audios": []}])
    got = m.forward(mi).logits.float()
    assert (got - ref).abs().max().item() < 2e-3 * max(ref.abs().max().item(), 1.0)


def test_qwen3_5_vision_tower_and_mrope_on_the_hybrid_decoder(tmp_path):
    """Qwen3.5 with a picture: the Qwen3-VL style tower without deep-stack outputs, interleaved M-RoPE on the
    rotary quarter of the full-attention heads, Gated DeltaNet layers in between, against
    Qwen3_5ForConditionalGeneration."""
    from transformers import Qwen3_5Config, Qwen3_5ForConditionalGeneration

    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.base import embed_row_width, load_config
    from lightllm_b200.models.registry import get_model, is_multimodal
    from lightllm_b200.models.vit.qwen2_vl_visual import patchify
    from lightllm_b200.models.vit.qwen3_vl_visual import Qwen3VLVisionTower
    from lightllm_b200.models.weights import SafetensorsSource
    from lightllm_b200.parallel import dist as pdist

    torch.manual_seed(0)
    text = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                num_key_value_heads=2, head_dim=64, vocab_size=300, linear_num_value_heads=4, linear_num_key_heads=2,
                linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4, full_attention_interval=2,
                max_position_embeddings=512,
                rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.25,
                                 "mrope_section": [2, 3, 3], "mrope_interleaved": True})
    vision = dict(depth=2, hidden_size=32, num_heads=4, intermediate_size=64, out_hidden_size=64, patch_size=16,
                  spatial_merge_size=2, temporal_patch_size=2, in_channels=3, num_position_embeddings=36,
                  hidden_act="gelu_pytorch_tanh")
    cfg = Qwen3_5Config(text_config=text, vision_config=vision, image_token_id=290, video_token_id=291,
                        vision_start_token_id=292, vision_end_token_id=293, tie_word_embeddings=False)
    hf = Qwen3_5ForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if ("norm" in n and "visual" not in n) or "dt_bias" in n or "A_log" in n:
                p.add_(torch.randn_like(p) * 0.1)
    d = str(tmp_path / "ckpt")
    hf.save_pretrained(d, safe_serialization=True)
    # the tensors under the names the modules have (model.language_model.*, model.visual.*), as released checkpoints
    from safetensors.torch import save_file
    save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, d + "/model.safetensors")

    pixels = torch.randn(1, 3, 64, 96)
    patches, (t, gh, gw) = patchify(pixels, patch=16)
    n_img = t * gh * gw // 4
    pre, post = [5, 17, 292], [293, 9, 44, 120, 7, 250, 31]
    hf_ids = torch.tensor([pre + [290] * n_img + post])
    with torch.no_grad():
        ref = hf(input_ids=hf_ids, pixel_values=patches, image_grid_thw=torch.tensor([[t, gh, gw]]),
                 mm_token_type_ids=(hf_ids == 290).long()).logits[0].float()
        vis = hf.model.visual(patches, grid_thw=torch.tensor([[t, gh, gw]]))

    conf = load_config(d)
    assert is_multimodal(conf) and embed_row_width(conf) == 64
    assert not is_multimodal({"model_type": "qwen3_5", "hidden_size": 64})       # a text-only checkpoint
    src = SafetensorsSource(d)
    tower = Qwen3VLVisionTower(conf["vision_config"], src, torch.device("cpu"), torch.float32)
    emb = tower.forward(patches, [(t, gh, gw)])
    assert emb.shape == (n_img, 64)
    assert (emb - vis.pooler_output).abs().max().item() < 1e-4

    class Arena:
        def read_rows(self, rows):
            return emb[rows - 40]

    m = get_model(conf, model_dir=d, pstate=pdist.ParallelState(device=torch.device("cpu")), data_type="float32",
                  max_total_token_num=256, max_req_num=2, max_seq_length=128, disable_cudagraph=True)
    assert type(m).__name__ == "Qwen3_5VLLM" and m.full_layers == [1, 3]
    m.embed_arena = Arena()
    tok0 = 100_000_000
    ids = torch.tensor(pre + list(range(tok0, tok0 + n_img)) + post)
    item = {"token_id": tok0, "token_num": n_img, "start_index_in_embed_cache": 40, "grid_thwd": (t, gh, gw, 2)}
    req, n = m.req_manager.alloc(), len(ids)
    mi = ModelInput(batch_size=1, total_token_num=n, max_kv_len=n, is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([n], dtype=torch.int32),
                    mem_indexes=m.mem_manager.alloc(n).clone(), input_ids=ids,
                    b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=n, return_all_logits=True,
                    multimodal_params=[{"images": [item], "audios": []}])
    got = m.forward(mi).logits.float()
    assert (got - ref).abs().max().item() < 2e-3 * max(ref.abs().max().item(), 1.0)


def test_tarsier2_llava_wrapper_over_qwen2_vl(tmp_path):
    """Tarsier2 checkpoints: `model_type: llava`, a Qwen2-VL decoder under `language_model.` and its tower under
    `vision_tower.`; same numbers as Qwen2-VL with the tensors renamed."""
    import json

    from safetensors.torch import save_file
    from transformers import Qwen2VLConfig, Qwen2VLForConditionalGeneration

    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.base import load_config
    from lightllm_b200.models.registry import get_model, is_multimodal
    from lightllm_b200.models.vit.qwen2_vl_visual import Qwen2VLVisionTower, patchify
    from lightllm_b200.models.weights import SafetensorsSource
    from lightllm_b200.parallel import dist as pdist

    torch.manual_seed(0)
    text = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                vocab_size=300, max_position_embeddings=512, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]})
    vision = dict(depth=2, embed_dim=32, hidden_size=64, num_heads=4, mlp_ratio=2, patch_size=14, spatial_merge_size=2,
                  temporal_patch_size=2, in_chans=3)
    hf = Qwen2VLForConditionalGeneration(Qwen2VLConfig(
        text_config=text, vision_config=vision, image_token_id=290, video_token_id=291, vision_start_token_id=292,
        vision_end_token_id=293)).eval().float()
    d = tmp_path / "ckpt"
    d.mkdir()
    renamed = {}
    for k, v in hf.state_dict().items():
        if k.startswith("model.language_model."):
            renamed["language_model.model." + k[len("model.language_model."):]] = v.contiguous()
        elif k.startswith("model.visual."):
            renamed["vision_tower." + k[len("model.visual."):]] = v.contiguous()
        elif k.startswith("lm_head."):
            renamed["language_model." + k] = v.contiguous()
    save_file(renamed, str(d / "model.safetensors"))
    wrapper = {"model_type": "llava", "architectures": ["LlavaForConditionalGeneration"],
               "text_config": dict(hf.config.text_config.to_dict(), model_type="qwen2_vl", image_token_id=290,
                                   vision_start_token_id=292, vision_end_token_id=293, tie_word_embeddings=False),
               "vision_config": dict(vision, model_type="qwen2_vl"), "image_token_index": 290}
    (d / "config.json").write_text(json.dumps(wrapper))

    pixels = torch.randn(1, 3, 56, 84)
    patches, (t, gh, gw) = patchify(pixels)
    n_img = t * gh * gw // 4
    pre, post = [5, 17, 292], [293, 9, 44, 120, 7]
    hf_ids = torch.tensor([pre + [290] * n_img + post])
    with torch.no_grad():
        ref = hf(input_ids=hf_ids, pixel_values=patches, image_grid_thw=torch.tensor([[t, gh, gw]]),
                 mm_token_type_ids=(hf_ids == 290).long()).logits[0].float()
    conf = load_config(str(d))
    assert is_multimodal(conf)
    tower = Qwen2VLVisionTower(conf["vision_config"], SafetensorsSource(str(d)), torch.device("cpu"), torch.float32,
                               prefix="vision_tower.")
    emb = tower.forward(patches, [(t, gh, gw)])

    class Arena:
        def read_rows(self, rows):
            return emb[rows - 40]

    m = get_model(conf, model_dir=str(d), pstate=pdist.ParallelState(device=torch.device("cpu")), data_type="float32",
                  max_total_token_num=256, max_req_num=2, max_seq_length=128, disable_cudagraph=True)
    assert type(m).__name__ == "Tarsier2Qwen2VLLM"
    m.embed_arena = Arena()
    tok0 = 100_000_000
    ids = torch.tensor(pre + list(range(tok0, tok0 + n_img)) + post)
    item = {"token_id": tok0, "token_num": n_img, "start_index_in_embed_cache": 40, "grid_thwd": (t, gh, gw, 2)}
    req, n = m.req_manager.alloc(), len(ids)
    mi = ModelInput(batch_size=1, total_token_num=n, max_kv_len=n, is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([n], dtype=torch.int32),
                    mem_indexes=m.mem_manager.alloc(n).clone(), input_ids=ids,
                    b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=n, return_all_logits=True,
                    multimodal_params=[{"images": [item], "audios": []}])
    got = m.forward(mi).logits.float()
    assert (got - ref).abs().max().item() < 2e-3 * max(ref.abs().max().item(), 1.0)


def test_qwen3_omni_thinker_audio_and_vision_towers(tmp_path):
    """Qwen3-Omni thinker with a picture and a sound clip in one prompt: audio tower (windowed convolutions, block
    attention), vision tower under the thinker's tensor names with deep-stack outputs, MoE decoder with interleaved
    M-RoPE, against Qwen3OmniMoeThinkerForConditionalGeneration."""
    import json

    from safetensors.torch import save_file
    from transformers.models.qwen3_omni_moe import modeling_qwen3_omni_moe as hfm
    from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeThinkerConfig

    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.base import embed_row_width, load_config
    from lightllm_b200.models.qwen3_omni import Qwen3OmniAudioTower, Qwen3OmniVisionTower, audio_token_num
    from lightllm_b200.models.registry import get_model, is_multimodal
    from lightllm_b200.models.vit.qwen2_vl_visual import patchify
    from lightllm_b200.models.weights import SafetensorsSource
    from lightllm_b200.parallel import dist as pdist

    torch.manual_seed(0)
    text = dict(hidden_size=64, intermediate_size=128, moe_intermediate_size=64, num_experts=4, num_experts_per_tok=2,
                num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=300,
                max_position_embeddings=512, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[],
                rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [2, 3, 3],
                                 "mrope_interleaved": True})
    vision = dict(depth=3, hidden_size=32, num_heads=4, intermediate_size=64, out_hidden_size=64, patch_size=16,
                  spatial_merge_size=2, temporal_patch_size=2, in_channels=3, num_position_embeddings=36,
                  deepstack_visual_indexes=[0, 2], hidden_act="gelu_pytorch_tanh")
    audio = dict(num_mel_bins=16, encoder_layers=2, encoder_attention_heads=2, encoder_ffn_dim=64, d_model=32,
                 max_source_positions=64, n_window=50, n_window_infer=200, output_dim=64, downsample_hidden_size=8,
                 conv_chunksize=500, activation_function="gelu")
    cfg = Qwen3OmniMoeThinkerConfig(text_config=text, vision_config=vision, audio_config=audio, audio_token_id=288,
                                    image_token_id=290, video_token_id=291, vision_start_token_id=292,
                                    vision_end_token_id=293, audio_start_token_id=294, audio_end_token_id=295,
                                    tie_word_embeddings=False)
    hf = hfm.Qwen3OmniMoeThinkerForConditionalGeneration(cfg).eval().float()
    d = tmp_path / "ckpt"
    d.mkdir()
    save_file({"thinker." + k: v.contiguous() for k, v in hf.state_dict().items()}, str(d / "model.safetensors"))
    (d / "config.json").write_text(json.dumps({"model_type": "qwen3_omni_moe", "thinker_config": cfg.to_dict()}))

    pixels = torch.randn(1, 3, 64, 96)
    patches, (t, gh, gw) = patchify(pixels, patch=16)
    n_img = t * gh * gw // 4
    frames = 337                                      # three full windows of 100 mel frames and a tail of 37
    mel = torch.randn(16, frames)
    n_aud = 3 * 13 + 5
    assert audio_token_num(frames * 160) == n_aud
    pre, mid, post = [5, 17, 292], [293, 9, 294], [295, 44, 120, 7]
    hf_ids = torch.tensor([pre + [290] * n_img + mid + [288] * n_aud + post])
    with torch.no_grad():
        ref = hf(input_ids=hf_ids, pixel_values=patches, image_grid_thw=torch.tensor([[t, gh, gw]]),
                 input_features=mel.unsqueeze(0), feature_attention_mask=torch.ones(1, frames, dtype=torch.long),
                 attention_mask=torch.ones_like(hf_ids)).logits[0].float()
        want_aud = hf.audio_tower(mel, feature_lens=torch.tensor([frames])).last_hidden_state
        vis = hf.visual(patches, grid_thw=torch.tensor([[t, gh, gw]]))

    conf = load_config(str(d))
    assert conf["model_type"] == "qwen3_omni_moe" and is_multimodal(conf) and embed_row_width(conf) == 192
    src = SafetensorsSource(str(d))
    atower = Qwen3OmniAudioTower(conf, src, torch.device("cpu"), torch.float32)
    aud = atower.forward(mel)
    assert aud.shape == (n_aud, 64) and (aud - want_aud).abs().max().item() < 1e-4
    assert set(Qwen3OmniAudioTower.weight_shapes(conf)) <= set(src.names())
    vtower = Qwen3OmniVisionTower(conf["vision_config"], src, torch.device("cpu"), torch.float32)
    emb = vtower.forward(patches, [(t, gh, gw)])
    assert (emb[:, :64] - vis.pooler_output).abs().max().item() < 1e-4
    assert set(Qwen3OmniVisionTower.weight_shapes(conf["vision_config"])) <= set(src.names())
    rows = torch.cat([emb, torch.nn.functional.pad(aud, (0, 128))], dim=0)   # arena: image rows, then audio rows

    class Arena:
        def read_rows(self, r):
            return rows[r - 40]

    m = get_model(conf, model_dir=str(d), pstate=pdist.ParallelState(device=torch.device("cpu")), data_type="float32",
                  max_total_token_num=256, max_req_num=2, max_seq_length=128, disable_cudagraph=True)
    assert type(m).__name__ == "Qwen3OmniThinkerLM"
    m.embed_arena = Arena()
    i0, a0 = 100_000_000, 100_001_000
    ids = torch.tensor(pre + list(range(i0, i0 + n_img)) + mid + list(range(a0, a0 + n_aud)) + post)
    image = {"token_id": i0, "token_num": n_img, "start_index_in_embed_cache": 40, "grid_thwd": (t, gh, gw, 2)}
    clip = {"token_id": a0, "token_num": n_aud, "start_index_in_embed_cache": 40 + n_img}
    req, n = m.req_manager.alloc(), len(ids)
    mi = ModelInput(batch_size=1, total_token_num=n, max_kv_len=n, is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([n], dtype=torch.int32),
                    mem_indexes=m.mem_manager.alloc(n).clone(), input_ids=ids,
                    b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=n, return_all_logits=True,
                    multimodal_params=[{"images": [image], "audios": [clip]}])
    got = m.forward(mi).logits.float()
    assert (got - ref).abs().max().item() < 2e-3 * max(ref.abs().max().item(), 1.0)


def _gemma4_check(tmp_path, cfg_kw, force_torch_attention=False, n_tokens=60):
    from transformers import Gemma4ForCausalLM, Gemma4TextConfig

    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.base import load_config
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.parallel import dist as pdist

    torch.manual_seed(0)
    cfg = Gemma4TextConfig(**cfg_kw)
    hf = Gemma4ForCausalLM(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n or "router.scale" in n or "per_expert_scale" in n:
                p.add_(torch.randn_like(p) * 0.1)
        for i, layer in enumerate(hf.model.layers):
            layer.layer_scalar.fill_(0.9 + 0.05 * i)
    d = str(tmp_path / "ckpt")
    hf.save_pretrained(d, safe_serialization=True)
    from safetensors.torch import save_file

    sd = {k: v.contiguous() for k, v in hf.state_dict().items()}
    if cfg.tie_word_embeddings:
        sd.pop("lm_head.weight", None)
    save_file(sd, d + "/model.safetensors")
    ids = torch.randint(3, cfg.vocab_size - 1, (n_tokens,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = hf(input_ids=ids.unsqueeze(0)).logits[0].float()
    m = get_model(load_config(d), model_dir=d, pstate=pdist.ParallelState(device=torch.device("cpu")),
                  data_type="float32", max_total_token_num=512, max_req_num=3, max_seq_length=128, disable_cudagraph=True)
    assert type(m).__name__ == "Gemma4TextLM"
    if force_torch_attention:
        m.big_head = 0
    scale = max(ref.abs().max().item(), 1.0)

    def prefill(req, tokens, ready):
        n = len(tokens)
        mi = ModelInput(batch_size=1, total_token_num=ready + n, max_kv_len=ready + n, is_prefill=True,
                        b_req_idx=torch.tensor([req], dtype=torch.int32),
                        b_seq_len=torch.tensor([ready + n], dtype=torch.int32),
                        mem_indexes=m.mem_manager.alloc(n).clone(), input_ids=tokens,
                        b_ready_cache_len=torch.tensor([ready], dtype=torch.int32), max_q_len=n, return_all_logits=True)
        return m.forward(mi).logits.float()

    r0 = m.req_manager.alloc()
    cut = n_tokens - 6
    got = torch.cat([prefill(r0, ids[:25], 0), prefill(r0, ids[25:cut], 25)])        # second chunk on a cached prefix
    assert (got - ref[:cut]).abs().max().item() < 2e-3 * scale
    for t in range(cut, n_tokens):
        m.req_manager.req_to_next_token_ids[r0] = int(ids[t])
        mi = ModelInput(batch_size=1, total_token_num=t + 1, max_kv_len=t + 1, is_prefill=False,
                        b_req_idx=torch.tensor([r0], dtype=torch.int32),
                        b_seq_len=torch.tensor([t + 1], dtype=torch.int32), mem_indexes=m.mem_manager.alloc(1).clone())
        step = m.forward(mi).logits.float()
        assert (step[0] - ref[t]).abs().max().item() < 2e-3 * scale, f"decode step at position {t}"
    return m


def test_gemma4_per_layer_inputs_shared_kv_and_k_eq_v(tmp_path):
    """Gemma-4 small-model features: two head sizes, proportional rotary embedding on global layers, V = K on global
    layers with fewer KV heads, the last layers reading earlier layers' caches with a double-wide MLP, per-layer
    inputs, layer scalars, logit soft-cap; sliding window shorter than the prompt."""
    kw = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=6, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, global_head_dim=32, num_global_key_value_heads=1,
              attention_k_eq_v=True, num_kv_shared_layers=2, use_double_wide_mlp=True, sliding_window=16,
              layer_types=["sliding_attention", "sliding_attention", "full_attention", "sliding_attention",
                           "sliding_attention", "full_attention"],
              hidden_size_per_layer_input=8, vocab_size_per_layer_input=300, final_logit_softcapping=30.0,
              max_position_embeddings=256, tie_word_embeddings=True, pad_token_id=0)
    m = _gemma4_check(tmp_path, kw)
    assert m.kv_src == [0, 1, 2, 3, 3, 2] and (m.n_pool_s, m.n_pool_g) == (3, 1)
    assert m.mem_manager.kv_sliding.shape[2:] == (4, 16) and m.mem_manager.kv_global.shape[2:] == (2, 32)


def test_gemma4_moe_block_and_torch_attention(tmp_path):
    """The mixture-of-experts block next to the dense MLP, and the torch attention used for head sizes above 256
    (forced here on small heads)."""
    kw = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, global_head_dim=32, sliding_window=12,
              layer_types=["sliding_attention", "sliding_attention", "full_attention"], hidden_size_per_layer_input=0,
              enable_moe_block=True, num_experts=4, top_k_experts=2, moe_intermediate_size=32,
              max_position_embeddings=256, tie_word_embeddings=False, pad_token_id=0)
    _gemma4_check(tmp_path, kw, force_torch_attention=True, n_tokens=40)


def test_gemma4_vision_tower_and_picture_tokens(tmp_path):
    """Gemma-4 with a picture: patch embedding with per-axis position tables, encoder blocks with two-axis rotary
    embedding, pooling by grid position, projection; soft tokens replace placeholder rows, per-layer inputs treat
    the placeholders as padding, picture tokens attend in both directions."""
    import json

    from safetensors.torch import save_file
    from transformers import Gemma4Config, Gemma4ForConditionalGeneration

    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.base import load_config
    from lightllm_b200.models.registry import get_model, is_multimodal
    from lightllm_b200.models.vit.gemma4_visual import Gemma4VisionTower, soft_token_num
    from lightllm_b200.models.weights import SafetensorsSource
    from lightllm_b200.parallel import dist as pdist

    torch.manual_seed(0)
    text = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                num_key_value_heads=2, head_dim=16, global_head_dim=32, sliding_window=16,
                layer_types=["sliding_attention", "sliding_attention", "full_attention"], hidden_size_per_layer_input=8,
                vocab_size_per_layer_input=300, max_position_embeddings=256, pad_token_id=0,
                use_bidirectional_attention="vision", tie_word_embeddings=True)
    vision = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=4, head_dim=8, patch_size=16, pooling_kernel_size=3, position_embedding_size=64,
                  use_clipped_linears=True, standardize=True)
    cfg = Gemma4Config(text_config=text, vision_config=vision, audio_config=None, image_token_id=290, boi_token_id=291,
                       eoi_token_id=292, video_token_id=293, audio_token_id=294)
    hf = Gemma4ForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n or "position_embedding_table" in n:
                p.add_(torch.randn_like(p) * 0.1)
        for n, b in hf.named_buffers():
            if n.endswith("input_min") or n.endswith("output_min"):
                b.fill_(-1.5)
            elif n.endswith("input_max") or n.endswith("output_max"):
                b.fill_(1.5)
            elif n.endswith("std_bias"):
                b.copy_(torch.randn_like(b) * 0.1)
            elif n.endswith("std_scale"):
                b.copy_(1 + torch.randn_like(b) * 0.1)
    d = tmp_path / "ckpt"
    d.mkdir()
    sd = {k: v.contiguous() for k, v in hf.state_dict().items() if k != "lm_head.weight"}
    save_file(sd, str(d / "model.safetensors"))
    (d / "config.json").write_text(json.dumps(cfg.to_dict()))

    conf = load_config(str(d))
    assert is_multimodal(conf) and soft_token_num(96, 96, 16, 4, 3) == 4
    tower = Gemma4VisionTower(conf, SafetensorsSource(str(d)), torch.device("cpu"), torch.float32)
    img = torch.rand(3, 96, 96)
    patches, pos = tower.patchify(img)
    assert patches.shape == (36, 768) and pos[7].tolist() == [1, 1]
    n_img = 4
    pre, post = [5, 17, 291], [292, 9, 44, 120, 7, 250]
    hf_ids = torch.tensor([pre + [290] * n_img + post])
    with torch.no_grad():
        feats = hf.model.get_image_features(patches.unsqueeze(0), pos.unsqueeze(0), return_dict=True).pooler_output
        ref = hf(input_ids=hf_ids, pixel_values=patches.unsqueeze(0), image_position_ids=pos.unsqueeze(0),
                 mm_token_type_ids=(hf_ids == 290).long()).logits[0].float()
    emb = tower.forward(patches, pos)
    assert emb.shape == (n_img, 64) and (emb - feats.reshape(n_img, 64)).abs().max().item() < 1e-4

    class Arena:
        def read_rows(self, rows):
            return emb[rows - 40]

    m = get_model(conf, model_dir=str(d), pstate=pdist.ParallelState(device=torch.device("cpu")), data_type="float32",
                  max_total_token_num=256, max_req_num=2, max_seq_length=128, disable_cudagraph=True)
    assert type(m).__name__ == "Gemma4LM" and m.bidirectional_pictures
    m.embed_arena = Arena()
    tok0 = 100_000_000
    ids = torch.tensor(pre + list(range(tok0, tok0 + n_img)) + post)
    item = {"token_id": tok0, "token_num": n_img, "start_index_in_embed_cache": 40}
    req, n = m.req_manager.alloc(), len(ids)
    mi = ModelInput(batch_size=1, total_token_num=n, max_kv_len=n, is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([n], dtype=torch.int32),
                    mem_indexes=m.mem_manager.alloc(n).clone(), input_ids=ids,
                    b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=n, return_all_logits=True,
                    multimodal_params=[{"images": [item], "audios": []}])
    got = m.forward(mi).logits.float()
    assert (got - ref).abs().max().item() < 2e-3 * max(ref.abs().max().item(), 1.0)


@pytest.mark.parametrize("kind", ["qwen2", "llama"])
def test_tarsier2_over_plain_decoders(tmp_path, kind):
    """Tarsier2 wrappers whose decoder is a plain Qwen2 / Llama model (sequential positions): the Qwen2-VL tower's
    embeddings replace the picture's run of ids; against the Hugging Face decoder fed with the same embeddings."""
    import json

    from safetensors.torch import save_file
    from transformers import LlamaConfig, LlamaForCausalLM, Qwen2Config, Qwen2ForCausalLM
    from transformers.models.qwen2_vl.configuration_qwen2_vl import Qwen2VLVisionConfig
    from transformers.models.qwen2_vl.modeling_qwen2_vl import Qwen2VisionTransformerPretrainedModel

    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.base import load_config
    from lightllm_b200.models.registry import get_model, is_multimodal
    from lightllm_b200.models.vit.qwen2_vl_visual import Qwen2VLVisionTower, patchify
    from lightllm_b200.models.weights import SafetensorsSource
    from lightllm_b200.parallel import dist as pdist
    from lightllm_b200.server.tokenizer import get_tokenizer

    torch.manual_seed(0)
    text = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                vocab_size=300, max_position_embeddings=512, tie_word_embeddings=False)
    vision = dict(depth=2, embed_dim=32, hidden_size=64, num_heads=4, mlp_ratio=2, patch_size=14, spatial_merge_size=2,
                  temporal_patch_size=2, in_chans=3)
    lm = (Qwen2ForCausalLM(Qwen2Config(**text)) if kind == "qwen2" else LlamaForCausalLM(LlamaConfig(**text))).eval().float()
    vit = Qwen2VisionTransformerPretrainedModel(Qwen2VLVisionConfig(**vision)).eval().float()
    d = tmp_path / "ckpt"
    d.mkdir()
    tensors = {"language_model." + k: v.contiguous() for k, v in lm.state_dict().items()}
    tensors.update({"vision_tower." + k: v.contiguous() for k, v in vit.state_dict().items()})
    save_file(tensors, str(d / "model.safetensors"))
    wrapper = {"model_type": "llava", "architectures": ["TarsierForConditionalGeneration"],
               "text_config": dict(lm.config.to_dict(), model_type=kind, image_token_id=290, vision_start_token_id=292,
                                   vision_end_token_id=293),
               "vision_config": dict(vision, model_type="qwen2_vl"), "image_token_index": 290}
    (d / "config.json").write_text(json.dumps(wrapper))

    pixels = torch.randn(1, 3, 56, 84)
    patches, (t, gh, gw) = patchify(pixels)
    n_img = t * gh * gw // 4
    pre, post = [5, 17, 292], [293, 9, 44, 120, 7]
    with torch.no_grad():
        feats = vit(patches, grid_thw=torch.tensor([[t, gh, gw]]))
        feats = getattr(feats, "pooler_output", feats)
        feats = feats[0] if isinstance(feats, (tuple, list)) else feats
        emb_in = lm.get_input_embeddings()(torch.tensor([pre + [0] * n_img + post]))
        emb_in[0, len(pre): len(pre) + n_img] = feats
        ref = lm(inputs_embeds=emb_in).logits[0].float()

    conf = load_config(str(d))
    assert is_multimodal(conf)
    tower = Qwen2VLVisionTower(conf["vision_config"], SafetensorsSource(str(d)), torch.device("cpu"), torch.float32,
                               prefix="vision_tower.")
    emb = tower.forward(patches, [(t, gh, gw)])
    assert (emb - feats).abs().max().item() < 1e-4

    class Arena:
        def read_rows(self, rows):
            return emb[rows - 40]

    m = get_model(conf, model_dir=str(d), pstate=pdist.ParallelState(device=torch.device("cpu")), data_type="float32",
                  max_total_token_num=256, max_req_num=2, max_seq_length=128, disable_cudagraph=True)
    assert type(m).__name__ == ("Tarsier2Qwen2LM" if kind == "qwen2" else "Tarsier2LlamaLM")
    m.embed_arena = Arena()
    tok0 = 100_000_000
    ids = torch.tensor(pre + list(range(tok0, tok0 + n_img)) + post)
    item = {"token_id": tok0, "token_num": n_img, "start_index_in_embed_cache": 40, "grid_thwd": (t, gh, gw, 2)}
    req, n = m.req_manager.alloc(), len(ids)
    mi = ModelInput(batch_size=1, total_token_num=n, max_kv_len=n, is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([n], dtype=torch.int32),
                    mem_indexes=m.mem_manager.alloc(n).clone(), input_ids=ids,
                    b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=n, return_all_logits=True,
                    multimodal_params=[{"images": [item], "audios": []}])
    got = m.forward(mi).logits.float()
    assert (got - ref).abs().max().item() < 2e-3 * max(ref.abs().max().item(), 1.0)

    # the serving tokenizer of such a checkpoint is the Qwen2-VL one, keyed by the wrapper's picture token
    tk = get_tokenizer(str(d), multimodal=True, vocab_size=300)
    assert type(tk).__name__ == "Qwen2VLTokenizer" and tk.image_pad_id == 290
