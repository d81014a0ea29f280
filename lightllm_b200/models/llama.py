"""Llama-family dense decoders: llama, mistral, qwen2 (qkv bias), qwen3 (q/k RMSNorm),
internlm2-style and other checkpoints that share the layer (reference: lightllm/models/llama,
qwen2, qwen3, mistral, internlm, stablelm, minicpm, phi3)."""
from __future__ import annotations

from .base import TransformerLM
from .registry import register_model


@register_model("llama", "mistral", "internlm3")
class LlamaLM(TransformerLM):
    model_type = "llama"


@register_model("qwen2")
class Qwen2LM(TransformerLM):
    model_type = "qwen2"

    def _read_config(self, c):
        super()._read_config(c)
        self.attn_bias = True


@register_model("qwen3")
class Qwen3LM(TransformerLM):
    model_type = "qwen3"

    def _read_config(self, c):
        super()._read_config(c)
        self.qk_norm = True
        self.attn_bias = c.get("attention_bias", False)
