"""InternVL: tile grid, tokenizer wrapper, and the InternViT tower + language model against the Hugging Face
implementation (its parameters renamed to the `internvl_chat` checkpoint layout)."""
import json
import os

import torch


def _to_internvl_chat(hf, layers):
    """HF InternVLForConditionalGeneration state dict -> `vision_model.* / mlp1.* / language_model.*` names."""
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    out = {}
    vt = "model.vision_tower."
    out["vision_model.embeddings.class_embedding"] = sd[vt + "embeddings.cls_token"]
    out["vision_model.embeddings.position_embedding"] = sd[vt + "embeddings.position_embeddings"]
    out["vision_model.embeddings.patch_embedding.weight"] = sd[vt + "embeddings.patch_embeddings.projection.weight"]
    out["vision_model.embeddings.patch_embedding.bias"] = sd[vt + "embeddings.patch_embeddings.projection.bias"]
    for i in range(layers):
        s, d = f"{vt}encoder.layer.{i}.", f"vision_model.encoder.layers.{i}."
        out[d + "attn.qkv.weight"] = torch.cat([sd[s + f"attention.{n}_proj.weight"] for n in "qkv"], 0)
        out[d + "attn.proj.weight"] = sd[s + "attention.projection_layer.weight"]
        out[d + "attn.proj.bias"] = sd[s + "attention.projection_layer.bias"]
        out[d + "attn.q_norm.weight"] = sd[s + "attention.q_norm.weight"]
        out[d + "attn.k_norm.weight"] = sd[s + "attention.k_norm.weight"]
        out[d + "ls1"], out[d + "ls2"] = sd[s + "lambda_1"], sd[s + "lambda_2"]
        for a, b in (("layernorm_before", "norm1"), ("layernorm_after", "norm2")):
            out[d + b + ".weight"], out[d + b + ".bias"] = sd[s + a + ".weight"], sd[s + a + ".bias"]
        for n in ("mlp.fc1.weight", "mlp.fc1.bias", "mlp.fc2.weight", "mlp.fc2.bias"):
            out[d + n] = sd[s + n]
    pj = "model.multi_modal_projector."
    for a, b in (("layer_norm", "0"), ("linear_1", "1"), ("linear_2", "3")):
        out[f"mlp1.{b}.weight"], out[f"mlp1.{b}.bias"] = sd[pj + a + ".weight"], sd[pj + a + ".bias"]
    for k, v in sd.items():
        if k.startswith("model.language_model."):
            out["language_model.model." + k[len("model.language_model."):]] = v
    out["language_model.lm_head.weight"] = sd["lm_head.weight"]
    return out


def test_tile_grid_and_token_count():
    from lightllm_b200.models.internvl import InternVLTokenizer
    from lightllm_b200.models.vit.internvl_visual import closest_grid, num_tiles
    from lightllm_b200.server.multimodal_params import ImageItem, MultimodalParams

    assert closest_grid(448, 448, 12) == (1, 1) and num_tiles(300, 200, 12) == 1
    assert closest_grid(1792, 448, 12) == (4, 1) and num_tiles(1792, 448, 12) == 5   # four tiles + thumbnail
    assert closest_grid(800, 1300, 6) in ((2, 3),) and num_tiles(800, 1300, 6) == 7
    assert num_tiles(4000, 4000, 6) <= 7

    class Tok:
        def convert_tokens_to_ids(self, t):
            return {"<img>": 250, "</img>": 251}[t]

        def encode(self, text, add_special_tokens=True):
            ids = []
            for w in text.replace("<img>", " <img> ").replace("</img>", " </img> ").split():
                ids.append({"<img>": 250, "</img>": 251}.get(w, 7))
            return ids

    tok = InternVLTokenizer(Tok(), {"vision_config": {"image_size": 448}})
    img = ImageItem(type="image_size", data=(1792, 448))
    img.image_w, img.image_h = 1792, 448
    mm = MultimodalParams.__new__(MultimodalParams)
    mm.images, mm.audios = [img], []
    tok.init_imageitem_extral_params(img, mm, None)
    assert img.extra_params["image_patch_max_num"] == 12
    assert tok.get_image_token_length(img) == 5 * 256
    img.token_id, img.token_num = 100_000_000, 5 * 256
    ids = tok.encode("look <image> here", mm)
    assert ids[:2] == [7, 250] and ids[2] == 100_000_000 and ids[2 + 1280] == 251 and len(ids) == 1280 + 4


def test_internvl_tower_and_language_model_match_hf(tmp_path):
    from safetensors.torch import save_file
    from transformers import InternVLConfig, InternVLForConditionalGeneration
    from transformers.models.internvl.configuration_internvl import InternVLVisionConfig

    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.base import load_config
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.models.vit.internvl_visual import InternVLVisionTower
    from lightllm_b200.models.weights import SafetensorsSource
    from lightllm_b200.parallel import dist as pdist

    torch.manual_seed(0)
    vc = InternVLVisionConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                              image_size=[56, 56], patch_size=[14, 14], use_qk_norm=True, norm_type="layer_norm",
                              layer_scale_init_value=0.5, use_mean_pooling=True)
    tc = dict(model_type="qwen2", hidden_size=96, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, vocab_size=300, max_position_embeddings=256, tie_word_embeddings=False)
    cfg = InternVLConfig(vision_config=vc, text_config=tc, image_token_id=290, downsample_ratio=0.5)
    hf = InternVLForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():  # layer scales and norms away from their trivial initial values
            if "lambda" in n or "norm" in n:
                p.add_(torch.randn_like(p) * 0.1)
    d = str(tmp_path / "ckpt")
    os.makedirs(d)
    save_file({k: v.contiguous() for k, v in _to_internvl_chat(hf, 2).items()}, os.path.join(d, "model.safetensors"))
    chat_cfg = {"model_type": "internvl_chat", "downsample_ratio": 0.5, "select_layer": -1, "ps_version": "v2",
                "vision_config": {"hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4,
                                  "intermediate_size": 128, "image_size": 56, "patch_size": 14,
                                  "qk_normalization": True, "norm_type": "layer_norm", "layer_norm_eps": 1e-6,
                                  "qkv_bias": False},
                "llm_config": {**tc, "architectures": ["Qwen2ForCausalLM"], "rms_norm_eps": 1e-6, "rope_theta": 10000.0}}
    json.dump(chat_cfg, open(os.path.join(d, "config.json"), "w"))

    pixels = torch.randn(2, 3, 56, 56)   # two tiles of one picture
    n_img = 2 * 4                        # (56 / 14)^2 / 4 tokens per tile
    pre, post = [5, 17, 250], [251, 9, 44]
    hf_ids = torch.tensor([pre + [290] * n_img + post])
    with torch.no_grad():
        ref = hf(input_ids=hf_ids, pixel_values=pixels).logits[0].float()
        want_emb = hf.model.get_image_features(pixels).pooler_output.reshape(n_img, -1)

    src = SafetensorsSource(d)
    tower = InternVLVisionTower(chat_cfg, src, torch.device("cpu"), torch.float32)
    assert tower.tokens_per_tile == 4
    emb = tower.forward(pixels).reshape(n_img, -1)
    assert (emb - want_emb).abs().max().item() < 1e-4
    assert set(InternVLVisionTower.weight_shapes(chat_cfg)) <= set(src.names())

    class Arena:
        def read_rows(self, rows):
            return emb[rows - 11]

    ps = pdist.ParallelState(device=torch.device("cpu"))
    m = get_model(load_config(d), model_dir=d, pstate=ps, data_type="float32", max_total_token_num=256, max_req_num=2,
                  max_seq_length=128, disable_cudagraph=True)
    assert type(m).__name__ == "InternVL_qwen2"
    m.embed_arena = Arena()
    tok0 = 100_000_000
    ids = torch.tensor(pre + list(range(tok0, tok0 + n_img)) + post)
    item = {"token_id": tok0, "token_num": n_img, "start_index_in_embed_cache": 11}
    req, n = m.req_manager.alloc(), len(ids)
    mi = ModelInput(batch_size=1, total_token_num=n, max_kv_len=n, is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([n], dtype=torch.int32),
                    mem_indexes=m.mem_manager.alloc(n).clone(), input_ids=ids,
                    b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=n, return_all_logits=True,
                    multimodal_params=[{"images": [item], "audios": []}])
    got = m.forward(mi).logits.float()
    assert (got - ref).abs().max().item() < 2e-3 * max(ref.abs().max().item(), 1.0)
