"""Qwen3-MoE (128 experts, top-8 softmax routing with renormalised weights, no shared expert), Qwen2-MoE
style shared experts, and Mixtral (8 experts, top-2).  Reference: lightllm/models/qwen3_moe, mixtral."""
from __future__ import annotations

from . import moe
from .base import TransformerLM
from .registry import register_model


@register_model("qwen3_moe")
class Qwen3MoeLM(TransformerLM):
    model_type = "qwen3_moe"
    gate_name, experts_name = "gate", "experts"

    def _read_config(self, c):
        super()._read_config(c)
        self.qk_norm = True
        self.attn_bias = c.get("attention_bias", False)
        self.moe = moe.MoEConfig(c["num_experts"], c["num_experts_per_tok"], c["moe_intermediate_size"],
                                 renorm=c.get("norm_topk_prob", True), act=self.act)
        self.ep = bool(self.extra.get("enable_ep_moe", False))
        step = c.get("decoder_sparse_step", 1)
        dense = set(c.get("mlp_only_layers", []) or [])
        self._moe_layers = {i for i in range(c["num_hidden_layers"]) if i not in dense and (i + 1) % step == 0}

    def _ffn_weight_shapes(self, p, layer):
        if layer in self._moe_layers:
            return moe.expert_weight_shapes(p + "mlp.", self.moe, self.hidden, self.gate_name, self.experts_name)
        return super()._ffn_weight_shapes(p, layer)

    def _load_ffn(self, lw, src, p, layer):
        if layer in self._moe_layers:
            moe.load_experts(self, lw, src, p + "mlp.", self.moe, self.ep, self.gate_name, self.experts_name)
        else:
            super()._load_ffn(lw, src, p, layer)

    def _ffn_block(self, i, lw, h, st):
        if lw.is_moe:
            return "partial", moe.moe_ffn(self, lw, h, self.moe, layer=i, st=st)
        return self._dense_ffn(lw, h)


@register_model("mixtral")
class MixtralLM(Qwen3MoeLM):
    model_type = "mixtral"

    def _read_config(self, c):
        c = dict(c)
        c.setdefault("num_experts", c.get("num_local_experts", 8))
        c.setdefault("moe_intermediate_size", c["intermediate_size"])
        c.setdefault("norm_topk_prob", True)
        TransformerLM._read_config(self, c)
        self.moe = moe.MoEConfig(c["num_experts"], c["num_experts_per_tok"], c["moe_intermediate_size"], renorm=True,
                                 act=self.act)
        self.ep = bool(self.extra.get("enable_ep_moe", False))
        self._moe_layers = set(range(c["num_hidden_layers"]))

    def _ffn_weight_shapes(self, p, layer):
        s = {p + "block_sparse_moe.gate.weight": (self.moe.num_experts, self.hidden)}
        for e in range(self.moe.num_experts):
            q = p + f"block_sparse_moe.experts.{e}."
            s[q + "w1.weight"] = (self.moe.inter, self.hidden)
            s[q + "w3.weight"] = (self.moe.inter, self.hidden)
            s[q + "w2.weight"] = (self.hidden, self.moe.inter)
        return s

    def _load_ffn(self, lw, src, p, layer):
        class _Rename:
            """Mixtral names (w1 = gate, w3 = up, w2 = down) presented under the common expert naming."""

            def __init__(self, base):
                self.base = base

            def _m(self, n):
                return (n.replace(".mlp.", ".block_sparse_moe.").replace("gate_proj", "w1").replace("up_proj", "w3")
                        .replace("down_proj", "w2"))

            def has(self, n):
                return self.base.has(self._m(n))

            def get(self, n, *a):
                return self.base.get(self._m(n), *a)

        moe.load_experts(self, lw, _Rename(src), p + "mlp.", self.moe, self.ep)
