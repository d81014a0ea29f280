"""LLaVA-1.5 style vision-language model: Llama (or Mistral) language model whose prompt carries one run of
virtual token ids per image; the embeddings come from the CLIP tower + projector in the visual server.
Reference: lightllm/models/llava.
"""
from __future__ import annotations

from .llama import LlamaLM
from .registry import register_model
from .remap import RemapSource


@register_model("llava", is_multimodal=True)
class LlavaLM(LlamaLM):
    model_type = "llava"

    def _wrap_source(self, src):
        if src.has("model.embed_tokens.weight"):
            return src
        t, used = {}, set()
        for pre, new in (("model.language_model.model.", "model."), ("language_model.model.", "model."),
                         ("model.language_model.", "model."), ("language_model.lm_head.", "lm_head."),
                         ("model.language_model.lm_head.", "lm_head.")):  # longest prefixes first
            for n in src.names():
                if n.startswith(pre) and n not in used:
                    used.add(n)
                    t[new + n[len(pre):]] = n
        return RemapSource(src, t) if t else src


class LlavaTokenizer:
    """Every `<image>` placeholder becomes the image's run of virtual token ids (fixed count per image)."""

    def __init__(self, tokenizer, model_cfg: dict):
        self.tokenizer = tokenizer
        vc = model_cfg.get("vision_config") or {}
        n = (vc.get("image_size", 336) // vc.get("patch_size", 14)) ** 2
        self.image_length = n if model_cfg.get("vision_feature_select_strategy", "default") == "default" else n + 1
        self.image_token_id = model_cfg.get("image_token_index", model_cfg.get("image_token_id", 32000))

    def __getattr__(self, name):
        return getattr(self.tokenizer, name)

    def init_imageitem_extral_params(self, img, multi_params=None, sampling_params=None):
        pass

    def get_image_token_length(self, img) -> int:
        return self.image_length

    def encode(self, prompt, multimodal_params=None, add_special_tokens: bool = True, **kw):
        ids = list(prompt) if isinstance(prompt, (list, tuple)) else \
            list(self.tokenizer.encode(prompt, add_special_tokens=add_special_tokens))
        images = list(multimodal_params.images) if multimodal_params is not None else []
        out, k = [], 0
        for t in ids:
            if t == self.image_token_id and k < len(images):
                out.extend(range(images[k].token_id, images[k].token_id + images[k].token_num))
                k += 1
            else:
                out.append(t)
        if k != len(images):
            raise ValueError(f"the prompt has {k} image placeholders for {len(images)} images")
        return out
