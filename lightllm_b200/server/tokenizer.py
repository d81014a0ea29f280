"""Tokenizer factory (HF fast / slow / auto) and the token-id-only stand-in used when a model
directory has no tokenizer files (synthetic benchmarks send token ids).
Reference: lightllm/server/tokenizer.py.
"""
from __future__ import annotations

import os
from typing import List


class IdOnlyTokenizer:
    """Accepts prompts that are already token ids; decodes ids as ``<id>`` strings."""

    eos_token_id = None
    all_special_ids: List[int] = []
    chat_template = None

    def __init__(self, vocab_size: int = 1 << 30):
        self.vocab_size = vocab_size

    def __len__(self):
        return self.vocab_size

    def encode(self, text, add_special_tokens=True):
        if isinstance(text, str):
            return [int(t) % self.vocab_size for t in text.split()] if text.replace(" ", "").isdigit() else \
                [ord(c) % self.vocab_size for c in text]
        return list(text)

    def decode(self, ids, skip_special_tokens=True, **kw):
        return "".join(f"<{int(i)}>" for i in ids)

    def convert_ids_to_tokens(self, ids, skip_special_tokens=False):
        if isinstance(ids, int):
            return f"<{ids}>"
        return [f"<{int(i)}>" for i in ids]

    def convert_tokens_to_string(self, tokens):
        return "".join(tokens)

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True, **kw):
        text = "".join(f"[{m.get('role', 'user')}]{m.get('content', '')}" for m in messages)
        return self.encode(text) if tokenize else text


def get_tokenizer(model_dir: str, tokenizer_mode: str = "fast", trust_remote_code: bool = False, vocab_size=None,
                  multimodal: bool = False, config_override: dict = None):
    tok = _get_text_tokenizer(model_dir, tokenizer_mode, trust_remote_code, vocab_size)
    if not multimodal:
        return tok
    from ..models.base import load_config

    cfg = config_override or load_config(model_dir)
    mt = cfg.get("model_type")
    from ..models.qwen2_vl import is_tarsier2

    if mt in ("qwen2_vl", "qwen2_5_vl") or is_tarsier2(cfg):
        from ..models.qwen2_vl import Qwen2VLTokenizer

        return Qwen2VLTokenizer(tok, cfg)
    if mt == "llava":
        from ..models.llava import LlavaTokenizer

        return LlavaTokenizer(tok, cfg)
    if mt in ("qwen3_vl", "qwen3_vl_moe", "qwen3_5", "qwen3_5_moe"):
        from ..models.qwen2_vl import Qwen3VLTokenizer

        return Qwen3VLTokenizer(tok, cfg)
    if mt == "qwen" and "visual" in cfg:
        from ..models.llama import QwenVLV1Tokenizer

        return QwenVLV1Tokenizer(tok, cfg)
    if mt == "qwen3_omni_moe":
        from ..models.qwen3_omni import Qwen3OmniTokenizer

        return Qwen3OmniTokenizer(tok, cfg)
    if mt == "gemma4":
        from ..models.gemma4 import Gemma4Tokenizer

        return Gemma4Tokenizer(tok, cfg)
    if mt == "gemma3":
        from ..models.generic import Gemma3Tokenizer

        return Gemma3Tokenizer(tok, cfg)
    if mt == "internvl_chat":
        from ..models.internvl import InternVLTokenizer

        return InternVLTokenizer(tok, cfg)
    raise ValueError(f"multimodal serving of model_type {mt!r} has no tokenizer wrapper")


def _get_text_tokenizer(model_dir: str, tokenizer_mode: str = "fast", trust_remote_code: bool = False, vocab_size=None):
    has_files = model_dir and any(os.path.exists(os.path.join(model_dir, f))
                                  for f in ("tokenizer.json", "tokenizer.model", "tokenizer_config.json", "vocab.json"))
    if not has_files:
        return IdOnlyTokenizer(vocab_size or (1 << 30))
    from transformers import AutoTokenizer

    use_fast = tokenizer_mode != "slow"
    try:
        tok = AutoTokenizer.from_pretrained(model_dir, use_fast=use_fast, trust_remote_code=trust_remote_code)
    except Exception:
        if tokenizer_mode == "auto" or use_fast:
            tok = AutoTokenizer.from_pretrained(model_dir, use_fast=not use_fast, trust_remote_code=trust_remote_code)
        else:
            raise
    if _model_type(model_dir) == "deepseek_v32":
        # no Jinja template ships with this model: its prompt format is rendered in Python
        from ..models.deepseek_v32_chat import DeepSeekV32Tokenizer

        tok = DeepSeekV32Tokenizer(tok)
    return tok


def _model_type(model_dir: str) -> str:
    try:
        import json

        with open(os.path.join(model_dir, "config.json")) as f:
            return str(json.load(f).get("model_type", ""))
    except (OSError, ValueError):
        return ""
