"""Llama-family dense decoders: llama, mistral, qwen2 (qkv bias), qwen3 (q/k RMSNorm),
internlm2-style and other checkpoints that share the layer (reference: lightllm/models/llama,
qwen2, qwen3, mistral, internlm, stablelm, minicpm, phi3)."""
from __future__ import annotations

import torch

from .base import TransformerLM
from .registry import register_model
from .remap import RemapSource, grouped_qkv, split_rows


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


@register_model("internlm")
class InternLM(TransformerLM):
    """Llama layer with biases on q/k/v/o (config key `bias`)."""

    def _read_config(self, c):
        super()._read_config(c)
        self.attn_bias = bool(c.get("bias", True))

    def _attn_weight_shapes(self, p):
        s = super()._attn_weight_shapes(p)
        if self.attn_bias:
            s[p + "self_attn.o_proj.bias"] = (self.hidden,)
        return s


@register_model("internlm2")
class InternLM2(TransformerLM):
    """Llama layer; the checkpoint fuses q/k/v per kv group (`attention.wqkv`) and names the MLP w1/w3/w2."""

    def _wrap_source(self, src):
        t = {"model.embed_tokens.weight": "model.tok_embeddings.weight", "lm_head.weight": "output.weight"}
        kv, g, D = self.num_kv_heads, self.num_q_heads // self.num_kv_heads, self.head_dim
        for i in range(self.num_layers):
            p = f"model.layers.{i}."
            t[p + "input_layernorm.weight"] = p + "attention_norm.weight"
            t[p + "post_attention_layernorm.weight"] = p + "ffn_norm.weight"
            for which in ("q", "k", "v"):
                t[f"{p}self_attn.{which}_proj.weight"] = grouped_qkv(p + "attention.wqkv.weight", kv, g, D, which)
            t[p + "self_attn.o_proj.weight"] = p + "attention.wo.weight"
            t[p + "mlp.gate_proj.weight"] = p + "feed_forward.w1.weight"
            t[p + "mlp.up_proj.weight"] = p + "feed_forward.w3.weight"
            t[p + "mlp.down_proj.weight"] = p + "feed_forward.w2.weight"
        return RemapSource(src, t)


@register_model("phi3")
class Phi3LM(TransformerLM):
    """Llama layer with fused `qkv_proj` and `gate_up_proj` tensors."""

    def _wrap_source(self, src):
        t = {}
        qd, kd = self.num_q_heads * self.head_dim, self.num_kv_heads * self.head_dim
        for i in range(self.num_layers):
            p = f"model.layers.{i}."
            t[p + "self_attn.q_proj.weight"] = split_rows(p + "self_attn.qkv_proj.weight", 0, qd)
            t[p + "self_attn.k_proj.weight"] = split_rows(p + "self_attn.qkv_proj.weight", qd, qd + kd)
            t[p + "self_attn.v_proj.weight"] = split_rows(p + "self_attn.qkv_proj.weight", qd + kd, qd + 2 * kd)
            t[p + "mlp.gate_proj.weight"] = split_rows(p + "mlp.gate_up_proj.weight", 0, self.inter)
            t[p + "mlp.up_proj.weight"] = split_rows(p + "mlp.gate_up_proj.weight", self.inter, 2 * self.inter)
        return RemapSource(src, t)


@register_model("minicpm")
class MiniCPM(TransformerLM):
    """Llama layer with muP-style scales: embeddings x scale_emb, every residual branch x scale_depth / sqrt(L)
    (folded into o_proj / down_proj at load), logits / (hidden / dim_model_base)."""

    def _read_config(self, c):
        super()._read_config(c)
        self.embed_scale = float(c.get("scale_emb", 1.0))
        self.branch_scale = float(c.get("scale_depth", 1.0)) / (self.num_layers ** 0.5)
        self.logit_scale = 1.0 / (self.hidden / float(c.get("dim_model_base", self.hidden)))

    def _load_attn(self, lw, src, p, layer):
        super()._load_attn(lw, src, p, layer)
        lw.o_w = (lw.o_w.float() * self.branch_scale).to(lw.o_w.dtype)

    def _load_ffn(self, lw, src, p, layer):
        super()._load_ffn(lw, src, p, layer)
        lw.down_w = (lw.down_w.float() * self.branch_scale).to(lw.down_w.dtype)


@register_model("qwen")
class QwenV1LM(TransformerLM):
    """First-generation Qwen: fused c_attn with bias, MLP out = c_proj(w1(x) * silu(w2(x))), config
    `intermediate_size` counts both halves."""

    def _read_config(self, c):
        c = dict(c)
        c["intermediate_size"] = c["intermediate_size"] // 2
        c.setdefault("rms_norm_eps", c.get("layer_norm_epsilon", 1e-6))
        c.setdefault("rope_theta", c.get("rotary_emb_base", 10000.0))
        c.setdefault("num_key_value_heads", c["num_attention_heads"])
        super()._read_config(c)
        self.attn_bias = True

    def _wrap_source(self, src):
        t = {"model.embed_tokens.weight": "transformer.wte.weight", "model.norm.weight": "transformer.ln_f.weight"}
        H = self.hidden
        for i in range(self.num_layers):
            p, q = f"model.layers.{i}.", f"transformer.h.{i}."
            t[p + "input_layernorm.weight"] = q + "ln_1.weight"
            t[p + "post_attention_layernorm.weight"] = q + "ln_2.weight"
            for k, name in enumerate(("q_proj", "k_proj", "v_proj")):
                t[f"{p}self_attn.{name}.weight"] = split_rows(q + "attn.c_attn.weight", k * H, (k + 1) * H)
                t[f"{p}self_attn.{name}.bias"] = split_rows(q + "attn.c_attn.bias", k * H, (k + 1) * H)
            t[p + "self_attn.o_proj.weight"] = q + "attn.c_proj.weight"
            t[p + "mlp.gate_proj.weight"] = q + "mlp.w2.weight"
            t[p + "mlp.up_proj.weight"] = q + "mlp.w1.weight"
            t[p + "mlp.down_proj.weight"] = q + "mlp.c_proj.weight"
        return RemapSource(src, t)


@register_model("qwen", condition=lambda cfg: "visual" in cfg, is_multimodal=True)
class QwenVLV1LM(QwenV1LM):
    """Qwen-VL (first generation): the Qwen decoder; the rows of picture placeholders are replaced by the resampler's
    256 embeddings per picture (`models/vit/qwen_vl_visual.py`).  Reference: lightllm/models/qwen_vl/model.py."""


class QwenVLV1Tokenizer:
    """`<img>anything</img>` in the prompt becomes `Picture k:<img>` + the k-th picture's id run + `</img>` + newline
    (reference: QWenVLTokenizer).  The ids of the two tags come from the tokenizer (`img_start_id`, `img_end_id`)."""

    def __init__(self, tokenizer, model_cfg: dict):
        self.tokenizer = tokenizer
        self.image_start_tag = getattr(tokenizer, "image_start_tag", "<img>")
        self.image_end_tag = getattr(tokenizer, "image_end_tag", "</img>")
        self.image_start_id = getattr(tokenizer, "img_start_id", model_cfg.get("img_start_id", 151857))
        self.image_end_id = getattr(tokenizer, "img_end_id", model_cfg.get("img_end_id", 151858))
        self.image_length = int((model_cfg.get("visual") or {}).get("n_queries", 256))

    def __getattr__(self, name):
        return getattr(self.tokenizer, name)

    def init_imageitem_extral_params(self, img, multi_params=None, sampling_params=None):
        pass

    def get_image_token_length(self, img) -> int:
        return self.image_length

    def _format_prompt(self, prompt: str) -> str:
        parts = prompt.split(self.image_start_tag)
        out = parts[0]
        for k, part in enumerate(parts[1:]):
            out += f"Picture {k + 1}:" + self.image_start_tag + part
        parts = out.split(self.image_end_tag)
        return parts[0] + "".join(self.image_end_tag + "\n" + part for part in parts[1:])

    def _encode_text(self, text: str):
        inner = getattr(self.tokenizer, "tokenizer", None)
        if inner is not None and hasattr(inner, "encode"):
            try:
                return list(inner.encode(text, allowed_special="all", disallowed_special=()))
            except TypeError:
                pass
        return list(self.tokenizer.encode(text))

    def encode(self, prompt, multimodal_params=None, **kw):
        import unicodedata

        if isinstance(prompt, (list, tuple)):
            ids = list(prompt)
        else:
            ids = self._encode_text(self._format_prompt(unicodedata.normalize("NFC", prompt)))
        images = list(multimodal_params.images) if multimodal_params is not None else []
        out, k, pos = [], 0, 0
        while True:
            try:
                s = ids.index(self.image_start_id, pos)
            except ValueError:
                break
            try:
                e = ids.index(self.image_end_id, s)
            except ValueError:
                raise ValueError("unclosed image tag") from None
            if k >= len(images):
                raise ValueError(f"the prompt has more image tags than the {len(images)} images sent")
            im = images[k]
            assert im.token_num == self.image_length, f"picture reserves {im.token_num} ids, the tower gives {self.image_length}"
            out.extend(ids[pos:s])
            out.append(self.image_start_id)
            out.extend(range(im.token_id, im.token_id + im.token_num))
            out.append(self.image_end_id)
            pos, k = e + 1, k + 1
        out.extend(ids[pos:])
        if k != len(images):
            raise ValueError(f"the prompt has {k} image tags for {len(images)} images")
        return out


@register_model("gemma")
class GemmaLM(TransformerLM):
    """Gemma (2B / 7B): RMSNorm with (1 + w), GeGLU, embeddings x sqrt(hidden), head size 256, tied lm_head."""

    def _read_config(self, c):
        super()._read_config(c)
        self.norm_w_offset = 1.0
        self.act = "gelu"
        self.embed_scale = float(torch.tensor(self.hidden ** 0.5, dtype=torch.bfloat16))
        self.tie_embeddings = True


class _RewardHead:
    """Reward models replace the vocabulary projection by a scalar score head on the last token; the forward
    pass returns it as a [B, 1] "logits" tensor that the reward backend stores in the request."""

    def _load_weights(self, src):
        super()._load_weights(src)
        self.lm_head_w = None
        self._load_score_head(src)

    def weight_shapes(self):
        s = super().weight_shapes()
        s.pop("lm_head.weight", None)
        s.update(self._score_shapes())
        return s

    def _lm_head(self, h, normed: bool = False):
        from .. import ops

        hn = h if normed else ops.rmsnorm(h, self.final_norm_w, self.eps, self.norm_w_offset)
        return self._score(hn)


@register_model("qwen2", condition=lambda c: "Qwen2ForRewardModel" in (c.get("architectures") or []))
class Qwen2RewardLM(_RewardHead, Qwen2LM):
    """Qwen2.5-Math-RM style: score = Linear(H, 1)(ReLU(Linear(H, H)(h))), both with bias
    (reference: lightllm/models/qwen2_reward)."""

    def _score_shapes(self):
        H = self.hidden
        return {"score.0.weight": (H, H), "score.0.bias": (H,), "score.2.weight": (1, H), "score.2.bias": (1,)}

    def _load_score_head(self, src):
        self.s0_w, self.s0_b = self._dev(src.get("score.0.weight")), self._dev(src.get("score.0.bias"))
        self.s2_w, self.s2_b = self._dev(src.get("score.2.weight")).float(), self._dev(src.get("score.2.bias")).float()

    def _score(self, hn):
        from .. import ops

        x = ops.gemm(hn, self.s0_w, bias=self.s0_b)
        ops.act_(x, "relu")
        return x.float() @ self.s2_w.t() + self.s2_b


@register_model("internlm2", condition=lambda c: "InternLM2ForRewardModel" in (c.get("architectures") or []))
class InternLM2RewardLM(_RewardHead, InternLM2):
    """InternLM2-reward: score = v_head(h), one Linear(H, 1) without bias (reference: lightllm/models/internlm2_reward)."""

    def _score_shapes(self):
        return {"v_head.weight": (1, self.hidden)}

    def _load_score_head(self, src):
        self.v_head_w = self._dev(src.get("v_head.weight")).float()

    def _score(self, hn):
        return hn.float() @ self.v_head_w.t()
