"""Probing of a HuggingFace model directory: config.json, dtype, eos ids, vocab size, the largest
sequence the model was trained for (rope scaling included).  Reference: lightllm/utils/config_utils.py.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional


def get_config_json(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg


def _text_cfg(cfg: dict) -> dict:
    for key in ("text_config", "llm_config", "language_config", "thinker_config"):
        if key in cfg and isinstance(cfg[key], dict):
            inner = cfg[key]
            if "text_config" in inner:
                inner = inner["text_config"]
            return {**cfg, **inner}
    return cfg


def get_eos_token_ids(model_dir: str) -> List[int]:
    cfg = _text_cfg(get_config_json(model_dir))
    e = cfg.get("eos_token_id")
    if e is None:
        gpath = os.path.join(model_dir, "generation_config.json")
        if os.path.exists(gpath):
            with open(gpath) as f:
                e = json.load(f).get("eos_token_id")
    if e is None:
        return []
    return list(e) if isinstance(e, (list, tuple)) else [e]


def get_vocab_size(model_dir: str) -> Optional[int]:
    cfg = _text_cfg(get_config_json(model_dir))
    return cfg.get("vocab_size")


def get_dtype(model_dir: str) -> str:
    cfg = _text_cfg(get_config_json(model_dir))
    dt = cfg.get("torch_dtype") or cfg.get("dtype") or "bfloat16"
    return str(dt).replace("torch.", "")


def get_model_max_len(model_dir: str, default: int = 16384) -> int:
    """max_position_embeddings x rope scaling factor (yarn / linear / dynamic), as the reference derives
    max_req_total_len when the flag is unset."""
    cfg = _text_cfg(get_config_json(model_dir))
    base = cfg.get("max_position_embeddings") or cfg.get("max_sequence_length") or cfg.get("seq_length")
    if base is None:
        return default
    rs = cfg.get("rope_scaling") or {}
    factor = 1.0
    kind = rs.get("rope_type", rs.get("type"))
    if kind in ("yarn", "linear", "dynamic") and "factor" in rs:
        orig = rs.get("original_max_position_embeddings")
        factor = float(rs["factor"])
        if orig:
            return int(orig * factor)
    return int(base * factor)


def has_shared_experts(model_dir: str) -> bool:
    cfg = _text_cfg(get_config_json(model_dir))
    return bool(cfg.get("n_shared_experts"))


def is_multimodal(model_dir: str) -> bool:
    cfg = get_config_json(model_dir)
    return any(k in cfg for k in ("vision_config", "visual", "audio_config")) or \
        cfg.get("model_type") in ("llava", "qwen2_vl", "qwen2_5_vl", "qwen3_vl", "internvl_chat", "gemma3")
