"""InternVL (`internvl_chat` checkpoints): an InternViT tower in the visual server plus one of several language
models (`llm_config.model_type`: internlm2, llama, qwen2, qwen3, phi3, qwen3_moe, deepseek_v2 / v3) whose weights
sit under `language_model.`.  The prompt marks every picture with `<image>`; the tokenizer wrapper turns it into
`<img>` + the picture's run of virtual token ids + `</img>`, one run of 256 ids per 448 x 448 tile.

Reference: lightllm/models/internvl/model.py (InternvlTokenizer and the per-LLM model classes).
"""
from __future__ import annotations

import os

from .registry import _REGISTRY, register_model
from .remap import RemapSource
from .vit.internvl_visual import num_tiles

IMG_START, IMG_END, IMG_TOKEN = "<img>", "</img>", "<image>"
AUDIO_START, AUDIO_END = "<audio>", "</audio>"


def _llm_type(cfg: dict) -> str:
    return (cfg.get("llm_config") or {}).get("model_type", "")


def _lift_llm_config(cfg: dict) -> dict:
    """The language model's settings at the top level (what the LM classes read), the wrapper's keys kept."""
    llm = dict(cfg.get("llm_config") or {})
    out = {**cfg, **llm}
    out["model_type"] = "internvl_chat"
    return out


class _InternVLMixin:
    """Loads the `language_model.*` weights of the checkpoint under the wrapped LM's own names."""

    def __init__(self, config: dict, **kw):
        super().__init__(_lift_llm_config(config), **kw)

    def _wrap_source(self, src):
        pre = "language_model."
        if not any(n.startswith(pre) for n in src.names()):
            return super()._wrap_source(src)
        inner = RemapSource(src, {n[len(pre):]: n for n in src.names() if n.startswith(pre)})
        return super()._wrap_source(inner)


def _register_variants():
    from . import _load_all  # noqa: F401  (the wrapped LM classes must be registered first)

    for llm in ("internlm2", "llama", "qwen2", "qwen3", "phi3", "qwen3_moe", "deepseek_v2", "deepseek_v3"):
        base = next((cls for cond, cls, _ in _REGISTRY.get(llm, []) if cond is None), None)
        if base is None:
            continue
        cls = type(f"InternVL_{llm}", (_InternVLMixin, base), {"model_type": "internvl_chat"})
        register_model("internvl_chat", condition=(lambda c, t=llm: _llm_type(c) == t), is_multimodal=True)(cls)


class InternVLTokenizer:
    """`<image>` -> `<img>` virtual ids `</img>`; the number of ids follows the picture's tile grid."""

    def __init__(self, tokenizer, model_cfg: dict):
        self.tokenizer = tokenizer
        self.image_length = int(os.environ.get("INTERNVL_IMAGE_LENGTH", 256))
        self.image_size = (model_cfg.get("vision_config") or {}).get("image_size", 448)
        self.use_thumbnail = bool(model_cfg.get("use_thumbnail", True))
        raw_conv = getattr(tokenizer, "convert_tokens_to_ids", None)

        def conv(tok):  # a vocabulary without the tag (text-only build of the model) gives None
            try:
                return raw_conv(tok)
            except (KeyError, ValueError):
                return None

        conv = conv if raw_conv else None
        self.image_start_id = conv(IMG_START) if conv else model_cfg.get("img_start_token_id")
        self.image_end_id = conv(IMG_END) if conv else model_cfg.get("img_end_token_id")
        self.image_token_id = model_cfg.get("image_token_id")  # id-list prompts: placeholder id of a picture
        self.audio_start_id = conv(AUDIO_START) if conv else model_cfg.get("audio_start_token_id")
        self.audio_end_id = conv(AUDIO_END) if conv else model_cfg.get("audio_end_token_id")

    def __getattr__(self, name):
        return getattr(self.tokenizer, name)

    def init_imageitem_extral_params(self, img, multi_params=None, sampling_params=None):
        """Tile budget of a picture: the request's `image_max_patch_num`, else MAX_PATCH_NUM, else by the number
        of pictures in the request (12 for one, 6 for up to six, a single tile beyond)."""
        want = getattr(sampling_params, "image_max_patch_num", -1) if sampling_params is not None else -1
        if want is not None and want > 0:
            img.extra_params["image_patch_max_num"] = int(want)
        elif os.getenv("MAX_PATCH_NUM"):
            img.extra_params["image_patch_max_num"] = int(os.getenv("MAX_PATCH_NUM"))
        else:
            n = len(multi_params.images) if multi_params is not None else 1
            img.extra_params["image_patch_max_num"] = 12 if n == 1 else (6 if n <= 6 else 0)

    def init_audioitem_extral_params(self, audio, multi_params=None, sampling_params=None):
        pass

    def get_audio_token_length(self, audio) -> int:
        from .whisper_audio import audio_token_num

        return audio_token_num(int(audio.audio_length))

    def get_image_token_length(self, img) -> int:
        cap = int(img.extra_params.get("image_patch_max_num", 12)) or 1
        return num_tiles(img.image_w, img.image_h, cap, self.image_size, self.use_thumbnail) * self.image_length

    def encode(self, prompt, multimodal_params=None, add_special_tokens: bool = True, **kw):
        images = list(multimodal_params.images) if multimodal_params is not None else []
        if isinstance(prompt, (list, tuple)):  # token ids: every `image_token_id` stands for one picture
            ids = list(prompt)
            out, k = [], 0
            for t in ids:
                if self.image_token_id is not None and t == self.image_token_id and k < len(images):
                    out += [self.image_start_id] if self.image_start_id is not None else []
                    out.extend(range(images[k].token_id, images[k].token_id + images[k].token_num))
                    out += [self.image_end_id] if self.image_end_id is not None else []
                    k += 1
                else:
                    out.append(t)
        else:
            text = prompt.replace(IMG_TOKEN, IMG_START + IMG_END, len(images))
            ids = list(self.tokenizer.encode(text, add_special_tokens=add_special_tokens))
            out, k, i = [], 0, 0
            while i < len(ids):
                if ids[i] == self.image_start_id and i + 1 < len(ids) and ids[i + 1] == self.image_end_id \
                        and k < len(images):
                    out.append(ids[i])
                    out.extend(range(images[k].token_id, images[k].token_id + images[k].token_num))
                    out.append(ids[i + 1])
                    k += 1
                    i += 2
                else:
                    out.append(ids[i])
                    i += 1
        if k != len(images):
            raise ValueError(f"invalid image tag num: {len(images)} images vs {k} placeholders")
        audios = list(multimodal_params.audios) if multimodal_params is not None else []
        if audios:  # `<audio></audio>` pairs of the prompt take the clips' virtual ids, in order
            ids, out, a, i = out, [], 0, 0
            while i < len(ids):
                if ids[i] == self.audio_start_id and i + 1 < len(ids) and ids[i + 1] == self.audio_end_id \
                        and a < len(audios):
                    out.append(ids[i])
                    out.extend(range(audios[a].token_id, audios[a].token_id + audios[a].token_num))
                    out.append(ids[i + 1])
                    a += 1
                    i += 2
                else:
                    out.append(ids[i])
                    i += 1
            if a != len(audios):
                raise ValueError(f"invalid audio tag num: {len(audios)} clips vs {a} placeholders")
        return out


_register_variants()
