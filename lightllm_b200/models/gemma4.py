"""Gemma-4 language model (text path of `gemma4` checkpoints and `gemma4_text`).

What differs from Gemma-3 and shapes this file:
* two kinds of attention layers with DIFFERENT head sizes: sliding-window layers (`head_dim`, default rotary
  base) and global layers (`global_head_dim`, "proportional" rotary embedding: only the first quarter of the
  rotary pairs turns, the rest has frequency zero; optionally fewer KV heads and V = the K projection before its
  norm, `attention_k_eq_v`).  The KV cache therefore has two pools that share the slot numbering;
* the last `num_kv_shared_layers` layers project no K / V: they read the cache of the last earlier layer of their
  kind (and, with `use_double_wide_mlp`, have a twice as wide MLP);
* q and k are RMS-normalised per head with a learned scale, v without one; attention scores are not scaled;
* RMSNorm multiplies by w (not 1 + w); sandwich norms around attention and MLP; an optional mixture-of-experts
  block runs NEXT TO the dense MLP on the same input (router: unscaled norm, learned per-channel scale, softmax,
  top-k renormalised, per-expert output scale) and the two normalised outputs are added;
* optional per-layer inputs: a second embedding table gives every layer a small vector per token, mixed with a
  projection of the main embedding; each layer gates it into the residual stream after its MLP;
* every layer output is multiplied by a stored scalar; logits may be soft-capped.

The projections, norms and expert GEMMs run on this package's kernels; the attention prologue (per-head norms,
rotary embedding, cache write) is torch glue because head sizes differ per layer; attention runs on the generic
kernel for head sizes up to 256 and on torch ops (per request, dense scores) above that, outside CUDA graphs.
`Gemma4LM` (bottom of the file) adds pictures: soft tokens of `models/vit/gemma4_visual.py` replace placeholder rows.
The audio tower of the small multimodal checkpoints is not built.

Reference: lightllm/models/gemma4/{model.py,layer_infer/transformer_layer_infer.py,layer_weights/*}.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from .. import ops
from ..common.mem_manager import MemoryManager
from ..ops import moe as moe_ops
from ..ops import reference as ref
from .base import LayerWeights, TransformerLM
from .registry import register_model
from .remap import RemapSource
from .weights import tp_range


class Gemma4MemoryManager(MemoryManager):
    """Two pools over one slot space: [sliding layers, slots, 2 * Hkv, D] and [global layers, slots, 2 * Hg, Dg].
    Only layers that own a cache are counted.  To the code that moves KV (staging pages of disaggregated serving,
    host / disk tiers) the manager looks like one layer whose row holds a token's elements of both pools."""

    def __init__(self, size, dtype, device, n_sliding, hkv, d, n_global, hg, dg):
        self.geo = (n_sliding, hkv, d, n_global, hg, dg)
        super().__init__(size, dtype, hkv, d, n_sliding + n_global, device)

    def _init_buffers(self):
        ns, hkv, d, ng, hg, dg = self.geo
        self.kv_sliding = torch.zeros((ns, self.size + 1, 2 * hkv, d), dtype=self.dtype, device=self.device)
        self.kv_global = torch.zeros((ng, self.size + 1, 2 * hg, dg), dtype=self.dtype, device=self.device)
        self.kv_buffer = self.kv_sliding          # for code that only asks where the cache lives
        # what everything that moves KV around sees: ONE layer whose row is a token's elements of both pools
        self.elems_s, self.elems_g = ns * 2 * hkv * d, ng * 2 * hg * dg
        self.layer_num = 1

    def kv_row_shape(self):
        return (self.elems_s + self.elems_g,)

    @staticmethod
    def bytes_per_token(dtype, n_sliding, hkv, d, n_global, hg, dg) -> int:
        return (n_sliding * 2 * hkv * d + n_global * 2 * hg * dg) * torch.empty((), dtype=dtype).element_size()

    def gather_pages(self, slots, out=None):
        """[1, n, elements of both pools] staging copy of the given slots."""
        idx = slots.to(self.device, torch.long)
        n = idx.shape[0]
        if out is None:
            out = torch.empty((1, n, self.elems_s + self.elems_g), dtype=self.dtype, device=self.device)
        row = torch.cat([self.kv_sliding[:, idx].permute(1, 0, 2, 3).reshape(n, -1),
                         self.kv_global[:, idx].permute(1, 0, 2, 3).reshape(n, -1)], dim=1)
        out[0, :n].copy_(row)
        return out

    def scatter_pages(self, slots, pages) -> None:
        idx = slots.to(self.device, torch.long)
        n = idx.shape[0]
        row = pages[0, :n].to(self.device)
        ns, rs, ds = self.kv_sliding.shape[0], self.kv_sliding.shape[2], self.kv_sliding.shape[3]
        ng, rg, dg = self.kv_global.shape[0], self.kv_global.shape[2], self.kv_global.shape[3]
        self.kv_sliding[:, idx] = row[:, : self.elems_s].reshape(n, ns, rs, ds).permute(1, 0, 2, 3)
        self.kv_global[:, idx] = row[:, self.elems_s:].reshape(n, ng, rg, dg).permute(1, 0, 2, 3)


def _rms(x, w: Optional[torch.Tensor], eps: float):
    """RMSNorm over the last axis in fp32, times w when given (no 1 + w)."""
    xf = x.float()
    y = xf * torch.pow(xf.pow(2).mean(-1, keepdim=True) + eps, -0.5)
    if w is not None:
        y = y * w.float()
    return y.to(x.dtype)


def _rope(x, cos, sin):
    """x [T, heads, D]; cos / sin [T, D / 2]; rotate-half pairs (i, i + D / 2)."""
    h = x.shape[-1] // 2
    xf = x.float()
    x1, x2 = xf[..., :h], xf[..., h:]
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


@register_model("gemma4_text", "gemma4")
class Gemma4TextLM(TransformerLM):
    model_type = "gemma4_text"
    supports_prefix_cache = True
    big_head = 256          # head sizes above this run the torch attention

    # ------------------------------------------------------------------ config
    def _read_config(self, c):
        c = dict(c)
        c.setdefault("hidden_act", c.get("hidden_activation", "gelu_pytorch_tanh"))
        super()._read_config(c)
        self.norm_w_offset = 0.0
        self.act = "gelu"
        self.embed_scale = float(torch.tensor(self.hidden ** 0.5, dtype=torch.bfloat16)) if self.dtype == torch.bfloat16 \
            else self.hidden ** 0.5
        self.tie_embeddings = c.get("tie_word_embeddings", True)
        n = self.num_layers
        types = c.get("layer_types") or ["sliding_attention" if (i + 1) % 6 else "full_attention" for i in range(n)]
        types = list(types)
        types[-1] = "full_attention"
        self.layer_types = types
        self.window = int(c.get("sliding_window") or 0)
        self.d_s = int(c.get("head_dim") or self.hidden // self.num_q_heads)
        self.d_g = int(c.get("global_head_dim") or self.d_s)
        self.k_eq_v = bool(c.get("attention_k_eq_v", False))
        self.hkv_all_s = int(c.get("num_key_value_heads") or self.num_q_heads)
        self.hkv_all_g = int(c.get("num_global_key_value_heads") or self.hkv_all_s) if self.k_eq_v else self.hkv_all_s
        tp = self.tp.size
        assert self.num_q_heads % tp == 0 and self.hkv_all_s % tp == 0 and self.hkv_all_g % tp == 0, \
            "attention heads must divide by the tensor-parallel size"
        self.hkv_s, self.hkv_g = self.hkv_all_s // tp, self.hkv_all_g // tp
        self.head_dim, self.hkv = self.d_s, self.hkv_s
        shared = int(c.get("num_kv_shared_layers") or 0)
        self.first_shared = n - shared if shared > 0 else n
        own = types[: self.first_shared]
        self.kv_src = []          # layer whose cache layer i reads
        for i, t in enumerate(types):
            if i < self.first_shared:
                self.kv_src.append(i)
            else:
                self.kv_src.append(len(own) - 1 - own[::-1].index(t))
        self.pool_idx = {}
        ks = kg = 0
        for i, t in enumerate(own):
            if t == "sliding_attention":
                self.pool_idx[i] = ("s", ks)
                ks += 1
            else:
                self.pool_idx[i] = ("g", kg)
                kg += 1
        self.n_pool_s, self.n_pool_g = ks, kg
        self.double_wide = bool(c.get("use_double_wide_mlp", False))
        self.pli = int(c.get("hidden_size_per_layer_input") or 0)
        self.pli_vocab = int(c.get("vocab_size_per_layer_input") or self.vocab)
        self.moe_on = bool(c.get("enable_moe_block", False))
        self.n_experts = int(c.get("num_experts") or 0)
        self.top_k = int(c.get("top_k_experts") or 0)
        self.moe_inter = int(c.get("moe_intermediate_size") or 0)
        self.logit_cap = float(c.get("final_logit_softcapping") or 0.0)
        self.pad_id = int(c.get("pad_token_id") or 0)
        self.bidirectional_pictures = c.get("use_bidirectional_attention") == "vision"
        rp = c.get("rope_parameters") or {}
        sl, fa = rp.get("sliding_attention") or {}, rp.get("full_attention") or {}
        self.theta_s = float(sl.get("rope_theta", 10000.0))
        self.theta_g = float(fa.get("rope_theta", 1000000.0))
        self.rope_type_g = fa.get("rope_type", "proportional")
        self.rope_frac_g = float(fa.get("partial_rotary_factor", 0.25 if self.rope_type_g == "proportional" else 1.0))
        self.rope_factor_g = float(fa.get("factor", 1.0))
        self.sm_scale = 1.0

    def _inter_of(self, i: int) -> int:
        return self.inter * (2 if self.double_wide and i >= self.first_shared else 1)

    def _geo(self, i: int):
        """(q heads, kv heads, head size) of layer i on this rank."""
        if self.layer_types[i] == "sliding_attention":
            return self.hq, self.hkv_s, self.d_s
        return self.hq, self.hkv_g, self.d_g

    # ------------------------------------------------------------------ weights
    def weight_shapes(self):
        H, L = self.hidden, self.num_layers
        s = {"model.embed_tokens.weight": (self.vocab, H), "model.norm.weight": (H,)}
        if not self.tie_embeddings:
            s["lm_head.weight"] = (self.vocab, H)
        if self.pli:
            s.update({"model.embed_tokens_per_layer.weight": (self.pli_vocab, L * self.pli),
                      "model.per_layer_model_projection.weight": (L * self.pli, H),
                      "model.per_layer_projection_norm.weight": (self.pli,)})
        for i in range(L):
            p = f"model.layers.{i}."
            glob = self.layer_types[i] != "sliding_attention"
            D = self.d_g if glob else self.d_s
            hkv = self.hkv_all_g if glob else self.hkv_all_s
            a = p + "self_attn."
            s.update({a + "q_proj.weight": (self.num_q_heads * D, H), a + "o_proj.weight": (H, self.num_q_heads * D),
                      a + "q_norm.weight": (D,), a + "k_norm.weight": (D,),
                      a + "k_proj.weight": (hkv * D, H)})
            if not (glob and self.k_eq_v):
                s[a + "v_proj.weight"] = (hkv * D, H)
            for nm in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm",
                       "post_feedforward_layernorm"):
                s[p + nm + ".weight"] = (H,)
            I = self._inter_of(i)
            s.update({p + "mlp.gate_proj.weight": (I, H), p + "mlp.up_proj.weight": (I, H),
                      p + "mlp.down_proj.weight": (H, I), p + "layer_scalar": (1,)})
            if self.pli:
                s.update({p + "per_layer_input_gate.weight": (self.pli, H), p + "per_layer_projection.weight": (H, self.pli),
                          p + "post_per_layer_input_norm.weight": (H,)})
            if self.moe_on:
                E, MI = self.n_experts, self.moe_inter
                s.update({p + "router.proj.weight": (E, H), p + "router.scale": (H,), p + "router.per_expert_scale": (E,),
                          p + "experts.gate_up_proj": (E, 2 * MI, H), p + "experts.down_proj": (E, H, MI)})
                for nm in ("post_feedforward_layernorm_1", "post_feedforward_layernorm_2", "pre_feedforward_layernorm_2"):
                    s[p + nm + ".weight"] = (H,)
        return s

    def _wrap_source(self, src):
        if src.has("model.embed_tokens.weight"):
            return src
        for pre in ("model.language_model.model.", "language_model.model.", "model.language_model."):
            if src.has(pre + "embed_tokens.weight"):
                t = {"model." + n[len(pre):]: n for n in src.names() if n.startswith(pre)}
                for head in ("lm_head.weight", "language_model.lm_head.weight"):
                    if src.has(head):
                        t["lm_head.weight"] = head
                return RemapSource(src, t)
        return src

    def _load_weights(self, src):
        tp, r = self.tp.size, self.tp.rank
        H = self.hidden
        emb = src.get("model.embed_tokens.weight")
        self.embed_w = self._dev(emb)
        self.embed_range = (0, self.vocab)
        self.final_norm_w = self._dev(src.get("model.norm.weight"))
        v0, v1 = tp_range(self.vocab, r, tp)
        if src.has("lm_head.weight") and not self.tie_embeddings:
            self.lm_head_w = self._dev(src.get("lm_head.weight", 0, v0, v1))
        else:
            self.lm_head_w = self._dev(emb[v0:v1]) if tp > 1 else self.embed_w
        if self.pli:
            self.pli_embed_w = self._dev(src.get("model.embed_tokens_per_layer.weight"))
            self.pli_proj_w = self._dev(src.get("model.per_layer_model_projection.weight"))
            self.pli_norm_w = self._dev(src.get("model.per_layer_projection_norm.weight"))
        h0, h1 = tp_range(self.num_q_heads, r, tp)
        self.layers = []
        for i in range(self.num_layers):
            lw = LayerWeights()
            p = f"model.layers.{i}."
            a = p + "self_attn."
            glob = self.layer_types[i] != "sliding_attention"
            D = self.d_g if glob else self.d_s
            k0, k1 = tp_range(self.hkv_all_g if glob else self.hkv_all_s, r, tp)
            lw.q_w = self._dev(src.get(a + "q_proj.weight", 0, h0 * D, h1 * D))
            lw.o_w = self._dev(src.get(a + "o_proj.weight", 1, h0 * D, h1 * D))
            lw.q_norm = self._dev(src.get(a + "q_norm.weight"))
            lw.k_norm = self._dev(src.get(a + "k_norm.weight"))
            lw.kv_w = None
            if i < self.first_shared:
                rows = [src.get(a + "k_proj.weight", 0, k0 * D, k1 * D)]
                if not (glob and self.k_eq_v):
                    rows.append(src.get(a + "v_proj.weight", 0, k0 * D, k1 * D))
                lw.kv_w = self._dev(torch.cat(rows, dim=0))
            for attr, nm in (("in_norm", "input_layernorm"), ("post_norm", "post_attention_layernorm"),
                             ("pre_ffn_norm", "pre_feedforward_layernorm"), ("post_ffn_norm", "post_feedforward_layernorm")):
                setattr(lw, attr, self._dev(src.get(p + nm + ".weight")))
            self._load_dense_ffn(lw, src, p + "mlp.", self._inter_of(i))
            lw.scalar = float(src.get(p + "layer_scalar").float().reshape(-1)[0]) if src.has(p + "layer_scalar") else 1.0
            if self.pli:
                lw.pli_gate_w = self._dev(src.get(p + "per_layer_input_gate.weight"))
                lw.pli_out_w = self._dev(src.get(p + "per_layer_projection.weight"))
                lw.pli_post_norm = self._dev(src.get(p + "post_per_layer_input_norm.weight"))
            if self.moe_on:
                MI = self.moe_inter
                m0, m1 = tp_range(MI, r, tp)
                lw.router_w = self._dev(src.get(p + "router.proj.weight"))
                lw.router_scale = src.get(p + "router.scale").to(self.device, torch.float32) * H ** -0.5
                lw.expert_scale = src.get(p + "router.per_expert_scale").to(self.device, torch.float32)
                gu = src.get(p + "experts.gate_up_proj")                       # [E, 2 MI, H]: gate rows, then up rows
                g, u = gu[:, m0:m1], gu[:, MI + m0:MI + m1]
                il = (m1 - m0) % ref.GATE_UP_BLOCK == 0
                lw.w13 = self._dev(ref.interleave_gate_up(g, u) if il else torch.cat([g, u], dim=1))
                lw.w13_interleaved = il
                lw.w2 = self._dev(src.get(p + "experts.down_proj")[:, :, m0:m1].contiguous())
                for attr, nm in (("post_ffn_norm_1", "post_feedforward_layernorm_1"),
                                 ("post_ffn_norm_2", "post_feedforward_layernorm_2"),
                                 ("pre_ffn_norm_2", "pre_feedforward_layernorm_2")):
                    setattr(lw, attr, self._dev(src.get(p + nm + ".weight")))
            self.layers.append(lw)

    # ------------------------------------------------------------------ rotary tables, memory
    def _init_rope(self):
        n = max(self.max_seq_length + 8, 16)
        pos = torch.arange(n, dtype=torch.float32, device=self.device)

        def table(inv):
            ang = pos[:, None] * inv[None, :].to(self.device)
            return ang.cos().contiguous(), ang.sin().contiguous()

        d = self.d_s
        inv_s = 1.0 / (self.theta_s ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
        self.cos_s, self.sin_s = table(inv_s)
        d = self.d_g
        if self.rope_type_g == "proportional":
            turning = int(self.rope_frac_g * d // 2)
            inv = 1.0 / (self.theta_g ** (torch.arange(0, 2 * turning, 2, dtype=torch.float32) / d))
            inv_g = torch.cat([inv, torch.zeros(d // 2 - turning)]) / self.rope_factor_g
        else:
            inv_g = 1.0 / (self.theta_g ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
        self.cos_g, self.sin_g = table(inv_g)
        self.cos, self.sin = self.cos_s, self.sin_s

    def kv_bytes_per_token(self):
        return Gemma4MemoryManager.bytes_per_token(self.dtype, self.n_pool_s, self.hkv_s, self.d_s, self.n_pool_g,
                                                   self.hkv_g, self.d_g)

    def _make_mem_manager(self, size):
        if max(self.d_s, self.d_g) > self.big_head:
            self.disable_cudagraph = True     # the torch attention reads lengths on the host
        return Gemma4MemoryManager(size, self.dtype, self.device, self.n_pool_s, self.hkv_s, self.d_s, self.n_pool_g,
                                   self.hkv_g, self.d_g)

    def _kv_layer(self, i: int):
        kind, k = self.pool_idx[self.kv_src[i]]
        mm = self.mem_manager
        return mm.kv_sliding[k] if kind == "s" else mm.kv_global[k]

    # ------------------------------------------------------------------ forward
    def _embed(self, ids, st):
        h = super()._embed(ids, st)
        if self.pli:
            L, P = self.num_layers, self.pli
            # picture / sound placeholders (virtual ids beyond the vocabulary) count as the padding token here
            pli_ids = torch.where(ids >= self.pli_vocab, torch.full_like(ids, self.pad_id), ids)
            tok = ops.embedding(pli_ids, self.pli_embed_w, 0, self.pli_vocab).view(-1, L, P).float() * P ** 0.5
            proj = (ops.gemm(h, self.pli_proj_w).float() * self.hidden ** -0.5).view(-1, L, P)
            proj = _rms(proj, self.pli_norm_w, self.eps).float()
            st.extra["per_layer_inputs"] = ((proj + tok.to(h.dtype).float()) * 2.0 ** -0.5).to(h.dtype)
        return h

    def _lm_head(self, h, normed: bool = False):
        hn = h if normed else ops.rmsnorm(h, self.final_norm_w, self.eps, 0.0)
        logits = self.tp.gather_logits(ops.gemm(hn, self.lm_head_w, epi="f32"))
        if self.logit_cap > 0:
            logits = torch.tanh(logits / self.logit_cap) * self.logit_cap
        return logits

    def _reduced(self, a, w):
        o = ops.gemm(a, w)
        if self.tp.size > 1:
            self.tp.all_reduce_(o)
        return o

    def _layers_forward(self, x, st):
        residual = x
        eps = self.eps
        pli = st.extra.get("per_layer_inputs") if self.pli else None
        for i, lw in enumerate(self.layers):
            h = ops.rmsnorm(residual, lw.in_norm, eps, 0.0)
            o = self._reduced(self._attention_block(i, lw, h, st), lw.o_w)
            residual = residual + ops.rmsnorm(o, lw.post_norm, eps, 0.0)
            h = ops.rmsnorm(residual, lw.pre_ffn_norm, eps, 0.0)
            _, act, down_w = self._dense_ffn(lw, h)
            m = self._reduced(act, down_w)
            if self.moe_on:
                m1 = ops.rmsnorm(m, lw.post_ffn_norm_1, eps, 0.0)
                m2 = ops.rmsnorm(self._experts(lw, residual), lw.post_ffn_norm_2, eps, 0.0)
                m = m1 + m2
            residual = residual + ops.rmsnorm(m, lw.post_ffn_norm, eps, 0.0)
            if pli is not None:
                g = ops.gemm(residual, lw.pli_gate_w)
                g = (F.gelu(g.float(), approximate="tanh") * pli[:, i].float()).to(residual.dtype)
                g = ops.gemm(g, lw.pli_out_w)
                residual = residual + ops.rmsnorm(g, lw.pli_post_norm, eps, 0.0)
            if lw.scalar != 1.0:
                residual = residual * lw.scalar
        return residual

    def _experts(self, lw, residual):
        x = residual
        r = _rms(x, None, self.eps).float() * lw.router_scale
        probs = torch.softmax(ops.gemm(r.to(x.dtype), lw.router_w).float(), dim=-1)
        w, idx = probs.topk(self.top_k, dim=-1)
        w = w / w.sum(-1, keepdim=True) * lw.expert_scale[idx]
        h2 = ops.rmsnorm(x, lw.pre_ffn_norm_2, self.eps, 0.0)
        if lw.w13_interleaved:
            out = moe_ops.fused_experts(h2, lw.w13, lw.w2, idx.to(torch.int32), w.float(), act="gelu")
        else:
            out = moe_ops.ref_fused_experts(h2, lw.w13, lw.w2, idx, w.float(), act="gelu", interleaved=False)
        if self.tp.size > 1:
            self.tp.all_reduce_(out)
        return out

    def _attention_block(self, i, lw, h, st):
        hq, hkv, D = self._geo(i)
        T = h.shape[0]
        glob = self.layer_types[i] != "sliding_attention"
        pos = st.position_ids.long()
        cos_t, sin_t = (self.cos_g, self.sin_g) if glob else (self.cos_s, self.sin_s)
        cos, sin = cos_t[pos], sin_t[pos]
        q = ops.gemm(h, lw.q_w).view(T, hq, D)
        q = _rope(_rms(q, lw.q_norm, self.eps), cos, sin)
        kv_layer = self._kv_layer(i)
        if lw.kv_w is not None:
            kv = ops.gemm(h, lw.kv_w)
            k = kv[:, : hkv * D].view(T, hkv, D)
            v = k if (glob and self.k_eq_v) else kv[:, hkv * D:].view(T, hkv, D)
            v = _rms(v, None, self.eps)
            k = _rope(_rms(k, lw.k_norm, self.eps), cos, sin)
            slot = st.mem_index.long()
            kv_layer[slot, :hkv] = k
            kv_layer[slot, hkv:] = v
        window = 0 if glob else self.window
        r2t = self.req_manager.req_to_token_indexs
        q2 = q.reshape(T, hq * D).contiguous()
        seq_pos = st.seq_pos
        if not glob and st.is_prefill and st.extra.get("seq_pos_pictures") is not None:
            seq_pos = st.extra["seq_pos_pictures"]
        if D <= self.big_head:
            o = ops.attention_generic(q2, kv_layer, r2t, st.b_req_idx, seq_pos,
                                      st.batch_of_token if st.is_prefill else None, hq, hkv, D, 1.0, window=window)
        else:
            o = self._attention_torch(q, kv_layer, r2t, st, hq, hkv, D, window)
        return o.reshape(T, hq * D)

    def _attention_torch(self, q, kv_layer, r2t, st, hq, hkv, D, window):
        """Per request: dense scores of its query tokens against its context under the causal / window mask."""
        dev = q.device
        B = st.b_req_idx.shape[0]
        reqs, lens = st.b_req_idx.tolist(), st.b_seq_len.tolist()
        q_len = st.extra["q_len_cpu"].tolist() if st.is_prefill else [1] * B
        G = hq // hkv
        out = torch.empty_like(q)
        off = 0
        for b in range(B):
            n, S = int(q_len[b]), int(lens[b])
            rows = kv_layer[r2t[reqs[b], :S].long()].float()                        # [S, 2 hkv, D]
            k = rows[:, :hkv].repeat_interleave(G, dim=1)
            v = rows[:, hkv:].repeat_interleave(G, dim=1)
            qpos = torch.arange(S - n, S, device=dev)
            kpos = torch.arange(S, device=dev)
            mask = kpos[None, :] <= qpos[:, None]
            if window > 0:
                mask &= kpos[None, :] > qpos[:, None] - window
            s = torch.einsum("thd,shd->hts", q[off:off + n].float(), k).masked_fill(~mask.unsqueeze(0), float("-inf"))
            out[off:off + n] = torch.einsum("hts,shd->thd", torch.softmax(s, dim=-1), v).to(q.dtype)
            off += n
        return out


@register_model("gemma4", condition=lambda cfg: bool(cfg.get("vision_config")), is_multimodal=True)
class Gemma4LM(Gemma4TextLM):
    """Gemma-4 with pictures: the soft tokens of the vision tower (`models/vit/gemma4_visual.py`) replace the
    placeholder rows (not scaled like word embeddings); with `use_bidirectional_attention: vision` the tokens of one
    picture see each other in both directions in the sliding-window layers (their causal limit becomes the
    picture's last position there; global layers stay causal).  The audio tower is not built."""

    def _prepare_prefill_state(self, st):
        super()._prepare_prefill_state(st)
        mm = st.extra.get("multimodal_params")
        if not mm or not self.bidirectional_pictures:
            return
        ids = st.extra["input_ids_cpu"]
        q_len = st.extra["q_len_cpu"].tolist()
        pos = st.seq_pos.clone()
        changed, off = False, 0
        for b, n_tok in enumerate(q_len):
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
            st.extra["seq_pos_pictures"] = pos      # used by the sliding-window layers only; global layers stay causal


class Gemma4Tokenizer:
    """Every image placeholder of the prompt (`<|image|>` text or its id) becomes begin-of-image id + the picture's
    virtual ids + end-of-image id; the number of ids follows the tower's resize rule."""

    def __init__(self, tokenizer, model_cfg: dict):
        self.tokenizer = tokenizer
        self.image_token = model_cfg.get("image_token", "<|image|>")
        self.image_token_id = model_cfg.get("image_token_id", 258_880)
        self.boi_id = model_cfg.get("boi_token_id", 255_999)
        self.eoi_id = model_cfg.get("eoi_token_id", 258_882)
        vc = model_cfg.get("vision_config") or {}
        self.patch = int(vc.get("patch_size", 16))
        self.k = int(vc.get("pooling_kernel_size", 3))
        self.max_soft_tokens = int(model_cfg.get("max_soft_tokens", 280))

    def __getattr__(self, name):
        return getattr(self.tokenizer, name)

    def init_imageitem_extral_params(self, img, multi_params=None, sampling_params=None):
        pass

    def get_image_token_length(self, img) -> int:
        from .vit.gemma4_visual import soft_token_num

        return soft_token_num(img.image_w, img.image_h, self.patch, self.max_soft_tokens, self.k)

    def encode(self, prompt, multimodal_params=None, add_special_tokens: bool = False, **kw):
        images = list(multimodal_params.images) if multimodal_params is not None else []

        def run(im):
            return [self.boi_id] + list(range(im.token_id, im.token_id + im.token_num)) + [self.eoi_id]

        out, k = [], 0
        if isinstance(prompt, (list, tuple)):
            for t in prompt:
                if t == self.image_token_id and k < len(images):
                    out += run(images[k])
                    k += 1
                else:
                    out.append(t)
        else:
            chunks = prompt.split(self.image_token)
            out = list(self.tokenizer.encode(chunks[0], add_special_tokens=add_special_tokens))
            for c in chunks[1:]:
                if k >= len(images):
                    raise ValueError("more image placeholders than pictures")
                out += run(images[k])
                k += 1
                out += list(self.tokenizer.encode(c, add_special_tokens=False))
        if k != len(images):
            raise ValueError(f"the prompt has {k} image placeholders for {len(images)} images")
        return out
