"""Chat prompt construction with the HF chat template (optionally overridden by --chat_template).
Reference: lightllm/server/build_prompt.py:129-164.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

_tokenizer = None
_template_override: Optional[str] = None


def init_tokenizer(tokenizer, chat_template_path: Optional[str] = None):
    global _tokenizer, _template_override
    _tokenizer = tokenizer
    if chat_template_path:
        with open(chat_template_path) as f:
            _template_override = f.read()


def _normalise(messages: List[Dict[str, Any]]):
    out = []
    for m in messages:
        m = dict(m)
        c = m.get("content")
        if isinstance(c, list):  # OpenAI content parts: keep the text, multimodal parts handled elsewhere
            m["content"] = "".join(p.get("text", "") for p in c if isinstance(p, dict) and p.get("type") == "text")
        out.append(m)
    return out


async def build_prompt(request, tools=None) -> str:
    messages = _normalise(request.messages)
    kwargs = {"conversation": messages}
    if request.character_settings:
        kwargs["character_settings"] = request.character_settings
    if request.role_settings:
        kwargs["role_setting"] = request.role_settings
    if request.chat_template_kwargs:
        kwargs.update(request.chat_template_kwargs)
    if tools:
        kwargs["tools"] = tools
    if _template_override:
        kwargs["chat_template"] = _template_override
    try:
        return _tokenizer.apply_chat_template(**kwargs, tokenize=False, add_generation_prompt=True)
    except TypeError:
        return _tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=True)
