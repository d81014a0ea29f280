"""Config-driven decoder for families outside the RMSNorm + gated-MLP + rotary mould: LayerNorm with bias,
plain (non-gated) MLPs, ALiBi or learned positions, partial rotary, sliding windows, sandwich norms.

The layer runs unfused (norm -> qkv GEMM -> rope/scatter -> attention -> o GEMM -> add+norm -> MLP GEMMs -> add+norm)
on this package's kernels; attention goes to the tensor-core kernels when the head size is 64 or 128 and nothing
but a causal mask is needed, else to the generic paged kernel (any head size <= 256, window / ALiBi / soft-cap).

Families: Bloom, StarCoder (GPT-BigCode), StarCoder2, StableLM, Gemma-3 text.
Reference: lightllm/models/{bloom,starcoder,starcoder2,stablelm,gemma3}.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .. import ops
from .base import LayerWeights, TransformerLM
from .registry import register_model
from .remap import RemapSource, per_head_qkv, split_rows
from .weights import WeightSource, tp_range


def alibi_slopes(n_heads: int) -> torch.Tensor:
    """Slopes of the ALiBi paper (geometric in the closest power of two, interleaved extension beyond it)."""
    p = 2 ** math.floor(math.log2(n_heads))
    base = 2.0 ** (-(2.0 ** -(math.log2(p) - 3)))
    s = [base ** (i + 1) for i in range(p)]
    if p != n_heads:
        extra_base = 2.0 ** (-(2.0 ** -(math.log2(2 * p) - 3)))
        s += [extra_base ** (2 * i + 1) for i in range(n_heads - p)]
    return torch.tensor(s, dtype=torch.float32)


class GenericDecoderLM(TransformerLM):
    model_type = "generic"

    # ------------------------------------------------------------------ config
    def _read_config(self, c):
        super()._read_config(c)
        self.norm_type = "rms"        # "rms" | "layer"
        self.norm_bias = False
        self.mlp_gated = True
        self.mlp_bias = False
        self.o_bias = False
        self.pos_type = "rope"        # "rope" | "alibi" | "learned"
        self.windows: List[int] = [0] * self.num_layers
        self.softcap = 0.0
        self.embed_norm = False
        self.sandwich = False         # norms on the attention / MLP outputs before the residual add (Gemma-3)
        self.act_name = {"gelu": "gelu", "gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh",
                         "gelu_fast": "gelu_tanh", "relu": "relu", "silu": "silu", "swish": "silu"}.get(
            str(c.get("hidden_act", c.get("hidden_activation", c.get("activation_function", "silu")))), "silu")
        self.max_pos = c.get("max_position_embeddings", c.get("n_positions", 2048))
        self.logit_scale = 1.0

    # ------------------------------------------------------------------ weights (canonical names)
    def _norm_shapes(self, name, n):
        s = {name + ".weight": (n,)}
        if self.norm_bias:
            s[name + ".bias"] = (n,)
        return s

    def weight_shapes(self) -> Dict[str, tuple]:
        H, D = self.hidden, self.head_dim
        s = {"model.embed_tokens.weight": (self.vocab, H)}
        s.update(self._norm_shapes("model.norm", H))
        if self.embed_norm:
            s.update(self._norm_shapes("model.embed_norm", H))
        if self.pos_type == "learned":
            s["model.pos_embed.weight"] = (self.max_pos, H)
        if not self.tie_embeddings:
            s["lm_head.weight"] = (self.vocab, H)
        for i in range(self.num_layers):
            p = f"model.layers.{i}."
            s.update(self._norm_shapes(p + "input_layernorm", H))
            s.update(self._norm_shapes(p + "post_attention_layernorm", H))
            if self.sandwich:
                s.update(self._norm_shapes(p + "pre_feedforward_layernorm", H))
                s.update(self._norm_shapes(p + "post_feedforward_layernorm", H))
            a = p + "self_attn."
            s[a + "q_proj.weight"] = (self.num_q_heads * D, H)
            s[a + "k_proj.weight"] = (self.num_kv_heads * D, H)
            s[a + "v_proj.weight"] = (self.num_kv_heads * D, H)
            s[a + "o_proj.weight"] = (H, self.num_q_heads * D)
            if self.attn_bias:
                s[a + "q_proj.bias"] = (self.num_q_heads * D,)
                s[a + "k_proj.bias"] = (self.num_kv_heads * D,)
                s[a + "v_proj.bias"] = (self.num_kv_heads * D,)
            if self.o_bias:
                s[a + "o_proj.bias"] = (H,)
            if self.qk_norm:
                s[a + "q_norm.weight"] = (D,)
                s[a + "k_norm.weight"] = (D,)
            m = p + "mlp."
            if self.mlp_gated:
                s[m + "gate_proj.weight"] = (self.inter, H)
            s[m + "up_proj.weight"] = (self.inter, H)
            s[m + "down_proj.weight"] = (H, self.inter)
            if self.mlp_bias:
                s[m + "up_proj.bias"] = (self.inter,)
                s[m + "down_proj.bias"] = (H,)
        return s

    def _get_norm(self, src, name):
        w = self._dev(src.get(name + ".weight"))
        b = self._dev(src.get(name + ".bias")) if (self.norm_bias and src.has(name + ".bias")) else None
        return w, b

    def _load_weights(self, src: WeightSource):
        tp, r = self.tp.size, self.tp.rank
        emb = src.get("model.embed_tokens.weight")
        self.embed_w = self._dev(emb)
        self.embed_range = (0, self.vocab)
        self.final_norm_w, self.final_norm_b = self._get_norm(src, "model.norm")
        if self.embed_norm:
            self.embed_norm_w, self.embed_norm_b = self._get_norm(src, "model.embed_norm")
        if self.pos_type == "learned":
            self.pos_embed_w = self._dev(src.get("model.pos_embed.weight"))
        v0, v1 = tp_range(self.vocab, r, tp)
        if src.has("lm_head.weight") and not self.tie_embeddings:
            self.lm_head_w = self._dev(src.get("lm_head.weight", 0, v0, v1))
        else:
            self.lm_head_w = self._dev(emb[v0:v1]) if tp > 1 else self.embed_w
        self.layers = []
        for i in range(self.num_layers):
            lw = LayerWeights()
            p = f"model.layers.{i}."
            lw.in_norm, lw.in_norm_b = self._get_norm(src, p + "input_layernorm")
            lw.post_norm, lw.post_norm_b = self._get_norm(src, p + "post_attention_layernorm")
            if self.sandwich:
                lw.pre_ffn_norm, _ = self._get_norm(src, p + "pre_feedforward_layernorm")
                lw.post_ffn_norm, _ = self._get_norm(src, p + "post_feedforward_layernorm")
            self._load_attn(lw, src, p, i)      # q/k/v (+bias, +q/k norm), o (+bias / tp)
            self._load_mlp(lw, src, p + "mlp.")
            self.layers.append(lw)
        if self.pos_type == "alibi":
            h0, h1 = tp_range(self.num_q_heads, r, tp)
            self.alibi = alibi_slopes(self.num_q_heads)[h0:h1].to(self.device)

    def _load_mlp(self, lw, src, m):
        tp, r = self.tp.size, self.tp.rank
        i0, i1 = tp_range(self.inter, r, tp)
        if self.mlp_gated:
            self._load_dense_ffn(lw, src, m, self.inter)
            return
        lw.up_w = self._dev(src.get(m + "up_proj.weight", 0, i0, i1))
        lw.down_w = self._dev(src.get(m + "down_proj.weight", 1, i0, i1))
        if self.mlp_bias:
            lw.up_b = self._dev(src.get(m + "up_proj.bias", 0, i0, i1))
            lw.down_b = self._dev(src.get(m + "down_proj.bias") / tp)

    # ------------------------------------------------------------------ forward
    def _norm(self, x, w, b=None):
        if self.norm_type == "layer":
            return ops.layernorm(x, w, b, self.eps)
        return ops.rmsnorm(x, w, self.eps, self.norm_w_offset)

    def _add_norm(self, residual, x, w, b=None):
        """residual += x; returns norm(residual)."""
        if self.norm_type == "layer":
            return ops.layernorm(x, w, b, self.eps, residual=residual)
        return ops.add_rmsnorm_(residual, x, w, self.eps, self.norm_w_offset)

    def _embed(self, ids, st):
        h = super()._embed(ids, st)
        if self.pos_type == "learned":
            h = h + ops.embedding(st.position_ids.to(torch.int64), self.pos_embed_w, 0, self.max_pos)
        if self.embed_norm:
            h = self._norm(h, self.embed_norm_w, self.embed_norm_b)
        return h

    def _lm_head(self, h):
        hn = self._norm(h, self.final_norm_w, self.final_norm_b)
        logits = ops.gemm(hn, self.lm_head_w, epi="f32")
        logits = self.tp.gather_logits(logits)
        return logits * self.logit_scale if self.logit_scale != 1.0 else logits

    def _reduced(self, a, w, bias):
        o = ops.gemm(a, w, bias=bias)
        if self.tp.size > 1:
            self.tp.all_reduce_(o)
        return o

    def _mlp(self, lw, h):
        if self.mlp_gated:
            _, act, down_w = self._dense_ffn(lw, h)
            return self._reduced(act, down_w, None)
        up = ops.gemm(h, lw.up_w, bias=lw.up_b)
        ops.act_(up, self.act_name)
        return self._reduced(up, lw.down_w, lw.down_b)

    def _layers_forward(self, x, st):
        residual = x
        n = self.num_layers
        h = self._norm(residual, self.layers[0].in_norm, self.layers[0].in_norm_b)
        for i, lw in enumerate(self.layers):
            a = self._attention_block(i, lw, h, st)
            o = self._reduced(a, lw.o_w, lw.o_b)
            if self.sandwich:
                o = self._norm(o, lw.post_norm)
                h = self._add_norm(residual, o, lw.pre_ffn_norm)
            else:
                h = self._add_norm(residual, o, lw.post_norm, lw.post_norm_b)
            m = self._mlp(lw, h)
            if self.sandwich:
                m = self._norm(m, lw.post_ffn_norm)
            if i + 1 < n:
                nxt = self.layers[i + 1]
                h = self._add_norm(residual, m, nxt.in_norm, nxt.in_norm_b)
            else:
                residual.add_(m)
        return residual

    def _rope_tables(self, i):
        return self.cos, self.sin

    def _attention_block(self, i, lw, h, st):
        D, hq, hkv = self.head_dim, self.hq, self.hkv
        qkv = ops.gemm(h, lw.qkv_w, bias=lw.qkv_b)
        kv_layer = self._kv_layer(i)
        cos, sin = self._rope_tables(i)
        ops.rope_kv_scatter_(qkv, kv_layer, cos, sin, st.position_ids, st.mem_index, hq, hkv, D,
                             self.rot_dim if self.pos_type == "rope" else 0, lw.q_norm, lw.k_norm, self.eps,
                             self.norm_w_offset)
        q = qkv[:, : hq * D]
        r2t = self.req_manager.req_to_token_indexs
        window = self.windows[i]
        alibi = self.alibi if self.pos_type == "alibi" else None
        plain = D in (64, 128) and window == 0 and alibi is None and self.softcap == 0.0
        if plain and st.is_prefill:
            o = ops.gqa_prefill(q, kv_layer, r2t, st.b_req_idx, st.cu_q, st.b_ready_cache_len, hq, hkv, D,
                                st.max_q_len, self.sm_scale)
        elif plain:
            o = ops.gqa_decode(q, kv_layer, r2t, st.b_req_idx, st.b_seq_len, hq, hkv, D, st.max_kv_len, self.sm_scale,
                               num_splits=st.decode_num_splits, scratch=st.decode_scratch)
        else:
            o = ops.attention_generic(q, kv_layer, r2t, st.b_req_idx, st.seq_pos,
                                      st.batch_of_token if st.is_prefill else None, hq, hkv, D, self.sm_scale,
                                      window=window, softcap=self.softcap, alibi=alibi)
        return o.view(-1, hq * D)


# ------------------------------------------------------------------------------------------------ families
@register_model("bloom")
class BloomLM(GenericDecoderLM):
    def _read_config(self, c):
        c = dict(c)
        c.setdefault("num_hidden_layers", c.get("n_layer"))
        c.setdefault("num_attention_heads", c.get("n_head"))
        c.setdefault("hidden_size", c.get("n_embed", c.get("hidden_size")))
        c.setdefault("intermediate_size", 4 * c["hidden_size"])
        c.setdefault("layer_norm_epsilon", 1e-5)
        super()._read_config(c)
        self.eps = c["layer_norm_epsilon"]
        self.norm_type, self.norm_bias = "layer", True
        self.mlp_gated, self.mlp_bias = False, True
        self.attn_bias = self.o_bias = True
        self.pos_type = "alibi"
        self.embed_norm = True
        self.tie_embeddings = True
        self.act_name = "gelu_tanh"

    def _wrap_source(self, src):
        t = {"model.embed_tokens.weight": "transformer.word_embeddings.weight",
             "model.embed_norm.weight": "transformer.word_embeddings_layernorm.weight",
             "model.embed_norm.bias": "transformer.word_embeddings_layernorm.bias",
             "model.norm.weight": "transformer.ln_f.weight", "model.norm.bias": "transformer.ln_f.bias"}
        nh, D = self.num_q_heads, self.head_dim
        for i in range(self.num_layers):
            p, q = f"model.layers.{i}.", f"transformer.h.{i}."
            for n in ("input_layernorm", "post_attention_layernorm"):
                for wb in ("weight", "bias"):
                    t[f"{p}{n}.{wb}"] = f"{q}{n}.{wb}"
            for k, name in enumerate(("q_proj", "k_proj", "v_proj")):
                t[f"{p}self_attn.{name}.weight"] = per_head_qkv(q + "self_attention.query_key_value.weight", nh, D, k)
                t[f"{p}self_attn.{name}.bias"] = per_head_qkv(q + "self_attention.query_key_value.bias", nh, D, k)
            for wb in ("weight", "bias"):
                t[f"{p}self_attn.o_proj.{wb}"] = f"{q}self_attention.dense.{wb}"
                t[f"{p}mlp.up_proj.{wb}"] = f"{q}mlp.dense_h_to_4h.{wb}"
                t[f"{p}mlp.down_proj.{wb}"] = f"{q}mlp.dense_4h_to_h.{wb}"
        return RemapSource(src, t)


@register_model("gpt_bigcode")
class StarcoderLM(GenericDecoderLM):
    def _read_config(self, c):
        c = dict(c)
        c.setdefault("num_hidden_layers", c.get("n_layer"))
        c.setdefault("num_attention_heads", c.get("n_head"))
        c.setdefault("hidden_size", c.get("n_embd"))
        c.setdefault("intermediate_size", c.get("n_inner") or 4 * c["hidden_size"])
        c["num_key_value_heads"] = 1 if c.get("multi_query", True) else c["num_attention_heads"]
        super()._read_config(c)
        self.eps = c.get("layer_norm_epsilon", 1e-5)
        self.norm_type, self.norm_bias = "layer", True
        self.mlp_gated, self.mlp_bias = False, True
        self.attn_bias = self.o_bias = True
        self.pos_type = "learned"
        self.tie_embeddings = True

    def _wrap_source(self, src):
        t = {"model.embed_tokens.weight": "transformer.wte.weight", "model.pos_embed.weight": "transformer.wpe.weight",
             "model.norm.weight": "transformer.ln_f.weight", "model.norm.bias": "transformer.ln_f.bias"}
        H, kvd = self.hidden, self.num_kv_heads * self.head_dim
        for i in range(self.num_layers):
            p, q = f"model.layers.{i}.", f"transformer.h.{i}."
            for wb in ("weight", "bias"):
                t[f"{p}input_layernorm.{wb}"] = f"{q}ln_1.{wb}"
                t[f"{p}post_attention_layernorm.{wb}"] = f"{q}ln_2.{wb}"
                t[f"{p}self_attn.q_proj.{wb}"] = split_rows(q + "attn.c_attn.", 0, H, wb)
                t[f"{p}self_attn.k_proj.{wb}"] = split_rows(q + "attn.c_attn.", H, H + kvd, wb)
                t[f"{p}self_attn.v_proj.{wb}"] = split_rows(q + "attn.c_attn.", H + kvd, H + 2 * kvd, wb)
                t[f"{p}self_attn.o_proj.{wb}"] = f"{q}attn.c_proj.{wb}"
                t[f"{p}mlp.up_proj.{wb}"] = f"{q}mlp.c_fc.{wb}"
                t[f"{p}mlp.down_proj.{wb}"] = f"{q}mlp.c_proj.{wb}"
        return RemapSource(src, t)


@register_model("starcoder2")
class Starcoder2LM(GenericDecoderLM):
    def _read_config(self, c):
        super()._read_config(c)
        self.eps = c.get("norm_epsilon", 1e-5)
        self.norm_type, self.norm_bias = "layer", True
        self.mlp_gated = False
        self.mlp_bias = self.attn_bias = self.o_bias = bool(c.get("use_bias", True))
        self.tie_embeddings = c.get("tie_word_embeddings", True)
        w = c.get("sliding_window") or 0
        self.windows = [int(w)] * self.num_layers

    def _wrap_source(self, src):
        t = {}
        for i in range(self.num_layers):
            p = f"model.layers.{i}.mlp."
            for wb in ("weight", "bias"):
                t[f"{p}up_proj.{wb}"] = f"{p}c_fc.{wb}"
                t[f"{p}down_proj.{wb}"] = f"{p}c_proj.{wb}"
        return RemapSource(src, t)


@register_model("stablelm")
class StableLM(GenericDecoderLM):
    def _read_config(self, c):
        super()._read_config(c)
        self.eps = c.get("layer_norm_eps", 1e-5)
        self.norm_type, self.norm_bias = "layer", True
        self.attn_bias = bool(c.get("use_qkv_bias", False))
        self.partial_rotary = c.get("partial_rotary_factor", c.get("rope_pct", 0.25))
        self.rot_dim = int(self.head_dim * self.partial_rotary)


@register_model("gemma3_text")
class Gemma3TextLM(GenericDecoderLM):
    """Gemma-3 language model: RMSNorm with (1 + w), q/k norm, sandwich norms, five sliding-window layers
    (local rotary base) per global layer, GeGLU, embeddings scaled by sqrt(hidden)."""

    def _read_config(self, c):
        super()._read_config(c)
        self.norm_w_offset = 1.0
        self.qk_norm = True
        self.sandwich = True
        self.act = "gelu"
        self.embed_scale = float(torch.tensor(self.hidden ** 0.5, dtype=torch.bfloat16))
        self.tie_embeddings = c.get("tie_word_embeddings", True)
        self.sm_scale = float(c.get("query_pre_attn_scalar", self.head_dim)) ** -0.5
        self.softcap = float(c.get("attn_logit_softcapping") or 0.0)
        w = int(c.get("sliding_window") or 0)
        types = c.get("layer_types")
        if types is None:
            pat = int(c.get("sliding_window_pattern", 6))
            types = ["full_attention" if (i + 1) % pat == 0 else "sliding_attention" for i in range(self.num_layers)]
        self.layer_types = types
        self.windows = [w if t == "sliding_attention" else 0 for t in types]
        rp = c.get("rope_parameters") or {}
        self.local_theta = float(c.get("rope_local_base_freq") or
                                 (rp.get("sliding_attention") or {}).get("rope_theta", 10000.0))
        if isinstance(rp.get("full_attention"), dict):
            self.rope_theta = float(rp["full_attention"].get("rope_theta", self.rope_theta))
            fa = rp["full_attention"]
            if fa.get("rope_type", "default") not in ("default", None):
                self.rope_scaling = {k: v for k, v in fa.items() if k != "rope_theta"}

    def _init_rope(self):
        from ..ops import reference as ref

        super()._init_rope()
        n = max(self.max_seq_length + 8, 16)
        self.cos_local, self.sin_local = ref.build_rope_cache(n, self.rot_dim, self.local_theta, None, device=self.device)

    def _rope_tables(self, i):
        if self.windows[i]:
            return self.cos_local, self.sin_local
        return self.cos, self.sin

    def _wrap_source(self, src):
        if src.has("model.embed_tokens.weight"):
            return src
        # multimodal checkpoints keep the text tower under language_model
        for pre in ("model.language_model.model.", "language_model.model.", "model.language_model."):
            if src.has(pre + "embed_tokens.weight"):
                t = {}
                for n in src.names() if hasattr(src, "names") else []:
                    if n.startswith(pre):
                        t["model." + n[len(pre):]] = n
                return RemapSource(src, t)
        return src


@register_model("gemma3", is_multimodal=True)
class Gemma3LM(Gemma3TextLM):
    """Gemma-3 with pictures: the SigLIP tower's 256 soft tokens per picture replace the placeholder rows (not
    scaled like word embeddings), and the tokens of one picture attend to each other in both directions: their
    causal limit is the picture's last position.  Reference: lightllm/models/gemma3/model.py (which keeps the
    picture tokens causal)."""

    def _prepare_prefill_state(self, st):
        super()._prepare_prefill_state(st)
        mm = st.extra.get("multimodal_params")
        if not mm:
            return
        ids = st.extra["input_ids_cpu"]
        q_len = st.extra["q_len_cpu"].tolist()
        pos = st.seq_pos.clone()
        changed, off = False, 0
        for b, n_tok in enumerate(q_len):  # per request: the same picture may appear in several requests of a batch
            params = mm[b] if b < len(mm) and mm[b] else {}
            seg = ids[off:off + n_tok]
            for it in params.get("images", []):
                t0, n = it.get("token_id"), it.get("token_num")
                if t0 is None:
                    continue
                hit = ((seg >= t0) & (seg < t0 + n)).nonzero(as_tuple=True)[0]
                if hit.numel() > 1:
                    hit = (hit + off).to(pos.device)
                    pos[hit] = pos[hit].max()
                    changed = True
            off += n_tok
        if changed:
            st.seq_pos = pos


class Gemma3Tokenizer:
    """`<start_of_image>` in the prompt becomes begin-of-image id + the picture's virtual ids + end-of-image id."""

    def __init__(self, tokenizer, model_cfg: dict):
        self.tokenizer = tokenizer
        self.boi_token, self.eoi_token = "<start_of_image>", "<end_of_image>"
        self.boi_id = model_cfg.get("boi_token_index", model_cfg.get("boi_token_id", 255_999))
        self.eoi_id = model_cfg.get("eoi_token_index", model_cfg.get("eoi_token_id", 256_000))
        self.image_token_id = model_cfg.get("image_token_index", model_cfg.get("image_token_id", 262_144))
        self.image_length = int(model_cfg.get("mm_tokens_per_image", 256))

    def __getattr__(self, name):
        return getattr(self.tokenizer, name)

    def init_imageitem_extral_params(self, img, multi_params=None, sampling_params=None):
        pass

    def get_image_token_length(self, img) -> int:
        return self.image_length

    def encode(self, prompt, multimodal_params=None, add_special_tokens: bool = False, **kw):
        images = list(multimodal_params.images) if multimodal_params is not None else []

        def run(im):
            return [self.boi_id] + list(range(im.token_id, im.token_id + im.token_num)) + [self.eoi_id]

        if isinstance(prompt, (list, tuple)):  # token ids: every image placeholder id stands for one picture
            out, k = [], 0
            for t in prompt:
                if t == self.image_token_id and k < len(images):
                    out += run(images[k])
                    k += 1
                else:
                    out.append(t)
        else:
            chunks = prompt.split(self.boi_token)
            out = list(self.tokenizer.encode(chunks[0], add_special_tokens=add_special_tokens))
            k = 0
            for c in chunks[1:]:
                if k >= len(images):
                    raise ValueError("more <start_of_image> tags than pictures")
                out += run(images[k])
                k += 1
                out += list(self.tokenizer.encode(c, add_special_tokens=False))
        if k != len(images):
            raise ValueError(f"the prompt has {k} image placeholders for {len(images)} images")
        return out
