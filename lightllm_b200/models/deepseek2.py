"""DeepSeek-V2 / V3 / R1 (and GLM-4.7-Flash, same layer): multi-head latent attention, a few dense
layers followed by MoE layers with routed + shared experts, sigmoid (V3) or softmax (V2) grouped
top-k routing with an optional score-correction bias, yarn RoPE with mscale.

KV pool row: [c_kv (kv_lora_rank, RMS-normalised) | k_pe (rotated)], one head, replicated over TP ranks.
Attention runs absorbed (see ops/mla.py): per layer
    q: x -> q_a_proj -> q_a_layernorm -> q_b_proj (heads sharded over TP)          [or q_proj]
    kv: x -> kv_a_proj_with_mqa (replicated) -> kv_a_layernorm on the latent, RoPE on k_pe -> pool
    q_lat = q_nope . W_UK (per head), MLA attention over the pool, o = o_lat . W_UV^T (per head), o_proj
W_UK / W_UV are the two halves of kv_b_proj, split per head at load time.  The de-interleaving that the
checkpoint's rotary layout needs is folded into the rows of q_b_proj / kv_a_proj at load time, so the
runtime RoPE is the plain half-split rotation.

fp8 checkpoints (e4m3 weights + `weight_scale_inv` 128x128 block scales) are accepted; see models/quant.py.

Reference: lightllm/models/deepseek2/* (model.py:75-115 yarn, layer_infer/transformer_layer_infer.py,
layer_weights/transformer_layer_weight.py), lightllm/models/glm4_moe_lite.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..common.mem_manager import MLAMemoryManager
from ..ops import mla as mla_ops
from ..ops import reference as ref
from ..ops.fp8 import Fp8Weight, interleave_gate_up_fp8
from . import moe, quant
from .base import TransformerLM
from .registry import register_model
from .weights import tp_range


def _yarn_mscale(scale: float, m: float) -> float:
    return 1.0 if scale <= 1 or not m else 0.1 * m * math.log(scale) + 1.0


def _deinterleave_rows(w: torch.Tensor, d: int) -> torch.Tensor:
    """Rows come in groups of d (one rotary head): reorder each group from (x0,y0,x1,y1,...) to (x0,x1,..,y0,y1,..)."""
    n = w.shape[0] // d
    idx = torch.arange(d).view(d // 2, 2).t().reshape(-1)
    return w.view(n, d, *w.shape[1:])[:, idx].reshape(w.shape)


@register_model("deepseek_v2", "deepseek_v3", "glm4_moe_lite", "kimi_k2")
class DeepseekV2LM(TransformerLM):
    model_type = "deepseek_v2"

    # ------------------------------------------------------------------ config
    def _read_config(self, c):
        super()._read_config(c)
        self.q_lora = c.get("q_lora_rank")
        self.kv_lora = c["kv_lora_rank"]
        self.nope = c["qk_nope_head_dim"]
        self.rope_d = c["qk_rope_head_dim"]
        self.v_dim = c["v_head_dim"]
        self.head_dim = self.nope + self.rope_d
        self.rot_dim = self.rope_d
        self.hkv = 1
        scale = (self.nope + self.rope_d) ** -0.5
        rs = c.get("rope_scaling") or {}
        if rs.get("mscale_all_dim"):
            m = _yarn_mscale(float(rs.get("factor", 1.0)), float(rs["mscale_all_dim"]))
            scale = scale * m * m
        self.sm_scale = scale
        self.first_dense = c.get("first_k_dense_replace", 0)
        self.moe_freq = c.get("moe_layer_freq", 1)
        n_routed = c.get("n_routed_experts")
        self.moe = None
        if n_routed:
            # V3-generation checkpoints route with sigmoid scores and a learned selection bias; configs written by
            # newer tooling omit the two keys that say so
            v3_like = c.get("model_type") in ("deepseek_v3", "deepseek_v32", "kimi_k2", "glm4_moe_lite")
            has_bias = c.get("topk_method", "noaux_tc" if v3_like else "greedy") == "noaux_tc"
            self.moe = moe.MoEConfig(n_routed, c["num_experts_per_tok"], c["moe_intermediate_size"],
                                     renorm=c.get("norm_topk_prob", True),
                                     scoring=c.get("scoring_func", "sigmoid" if v3_like else "softmax"), n_group=c.get("n_group") or 1,
                                     topk_group=c.get("topk_group") or 1,
                                     routed_scale=float(c.get("routed_scaling_factor", 1.0)), has_bias=has_bias,
                                     n_shared=c.get("n_shared_experts") or 0,
                                     shared_inter=c["moe_intermediate_size"] * (c.get("n_shared_experts") or 0),
                                     act=self.act)
        self.ep = bool(self.extra.get("enable_ep_moe", False))
        self.fp8 = quant.is_fp8_block_config(c) or str(self.extra.get("quant_type", "none")).startswith("fp8w8a8-b128")
        # fp8 checkpoints run their big matrices (experts, dense FFN, q_b, o_proj) on the block-scaled fp8 GEMM;
        # dequant_fp8=True keeps the older load path that expands everything to bf16
        self.fp8_compute = self.fp8 and not self.extra.get("dequant_fp8", False)

    def _is_moe_layer(self, i):
        return self.moe is not None and i >= self.first_dense and i % self.moe_freq == 0

    # ------------------------------------------------------------------ weights
    def fp8_weight_names(self):
        if not self.fp8:
            return set()
        return {n for n in self.weight_shapes() if n.endswith("proj.weight") and "kv_a_proj" not in n and
                "scale_inv" not in n}

    def _attn_weight_shapes(self, p):
        H = self.hidden
        s = {}
        qdim = self.num_q_heads * (self.nope + self.rope_d)
        if self.q_lora:
            s[p + "self_attn.q_a_proj.weight"] = (self.q_lora, H)
            s[p + "self_attn.q_a_layernorm.weight"] = (self.q_lora,)
            s[p + "self_attn.q_b_proj.weight"] = (qdim, self.q_lora)
        else:
            s[p + "self_attn.q_proj.weight"] = (qdim, H)
        s[p + "self_attn.kv_a_proj_with_mqa.weight"] = (self.kv_lora + self.rope_d, H)
        s[p + "self_attn.kv_a_layernorm.weight"] = (self.kv_lora,)
        s[p + "self_attn.kv_b_proj.weight"] = (self.num_q_heads * (self.nope + self.v_dim), self.kv_lora)
        s[p + "self_attn.o_proj.weight"] = (H, self.num_q_heads * self.v_dim)
        return s

    def _ffn_weight_shapes(self, p, layer):
        if self._is_moe_layer(layer):
            return moe.expert_weight_shapes(p + "mlp.", self.moe, self.hidden)
        return super()._ffn_weight_shapes(p, layer)

    def weight_shapes(self):
        s = super().weight_shapes()
        if self.fp8:
            extra = {}
            for n, shp in s.items():
                if n.endswith("proj.weight") and len(shp) == 2 and "kv_a_proj" not in n:
                    extra[n + "_scale_inv"] = ((shp[0] + 127) // 128, (shp[1] + 127) // 128)
            s.update(extra)
        return s

    def _w(self, src, name, dim=None, start=0, end=None):
        """bf16 view of a (possibly fp8 block-quantised) checkpoint tensor slice."""
        return quant.load_dequant(src, name, dim, start, end, self.dtype)

    def _load_attn(self, lw, src, p, layer):
        tp, r = self.tp.size, self.tp.rank
        h0, h1 = tp_range(self.num_q_heads, r, tp)
        qd = self.nope + self.rope_d
        a = p + "self_attn."

        def fix_q(w):  # de-interleave the rope part of every head
            w = w.view(-1, qd, w.shape[-1]).clone()
            w[:, self.nope:] = _deinterleave_rows(w[:, self.nope:].reshape(-1, w.shape[-1]), self.rope_d).view(
                -1, self.rope_d, w.shape[-1])
            return w.view(-1, w.shape[-1])

        def load_q(name):
            # the rope rows of a head are 64 rows starting at a multiple of 64, so they stay inside one 128-row
            # scale block and the fp8 payload can be permuted without touching the scales
            if self.fp8_compute and (h0 * qd) % 128 == 0 and self.nope % 64 == 0 and self.rope_d == 64:
                fw = quant.load_fp8_weight(src, name, 0, h0 * qd, h1 * qd)
                q8 = fix_q(fw.q.view(torch.uint8)).view(torch.float8_e4m3fn)
                return Fp8Weight(q8, fw.scale, 128).to(self.device)
            return self._dev(fix_q(self._w(src, name, 0, h0 * qd, h1 * qd)))

        if self.q_lora:
            lw.q_a_w = self._dev(self._w(src, a + "q_a_proj.weight"))
            lw.q_a_norm = self._dev(src.get(a + "q_a_layernorm.weight"))
            lw.q_b_w = load_q(a + "q_b_proj.weight")
        else:
            lw.q_b_w = load_q(a + "q_proj.weight")
        kva = self._w(src, a + "kv_a_proj_with_mqa.weight").clone()
        kva[self.kv_lora:] = _deinterleave_rows(kva[self.kv_lora:], self.rope_d)
        if self.q_lora:  # one GEMM produces the q latent and the kv latent
            lw.qkv_a_w = self._dev(torch.cat([self._w(src, a + "q_a_proj.weight"), kva], dim=0))
            lw.q_a_w = None
        else:
            lw.kv_a_w = self._dev(kva)
        lw.kv_a_norm = self._dev(src.get(a + "kv_a_layernorm.weight"))
        kvb = self._w(src, a + "kv_b_proj.weight", 0, h0 * (self.nope + self.v_dim), h1 * (self.nope + self.v_dim))
        kvb = kvb.view(h1 - h0, self.nope + self.v_dim, self.kv_lora)
        # W_UK as [h, kv_lora, nope] (q_lat = q_nope . W_UK: contraction over nope), W_UV as [h, v, kv_lora]
        lw.w_uk = self._dev(kvb[:, : self.nope].transpose(1, 2))
        lw.w_uv = self._dev(kvb[:, self.nope:])
        if self.fp8_compute and (h0 * self.v_dim) % 128 == 0:
            lw.o_w = quant.load_fp8_weight(src, a + "o_proj.weight", 1, h0 * self.v_dim, h1 * self.v_dim).to(self.device)
        else:
            lw.o_w = self._dev(self._w(src, a + "o_proj.weight", 1, h0 * self.v_dim, h1 * self.v_dim))

    def _load_dense_ffn(self, lw, src, prefix, inter, tp=None, r=None):
        raw = getattr(src, "base", src)
        tp_ = self.tp.size if tp is None else tp
        r_ = self.tp.rank if r is None else r
        i0, i1 = tp_range(inter, r_, tp_)
        if self.fp8_compute and i0 % 128 == 0 and (i1 - i0) % 128 == 0 and self.act == "silu":
            g = quant.load_fp8_weight(raw, prefix + "gate_proj.weight", 0, i0, i1)
            u = quant.load_fp8_weight(raw, prefix + "up_proj.weight", 0, i0, i1)
            lw.gate_up_w = interleave_gate_up_fp8(g, u).to(self.device)
            lw.gate_up_fused = True
            lw.down_w = quant.load_fp8_weight(raw, prefix + "down_proj.weight", 1, i0, i1).to(self.device)
            return
        super()._load_dense_ffn(lw, quant.DequantSource(raw, self.dtype) if self.fp8 else raw, prefix, inter, tp, r)

    def _load_ffn(self, lw, src, p, layer):
        if self._is_moe_layer(layer):
            moe.load_experts(self, lw, quant.DequantSource(src, self.dtype) if self.fp8 else src, p + "mlp.", self.moe,
                             self.ep)
        else:
            super()._load_ffn(lw, src, p, layer)

    # ------------------------------------------------------------------ memory
    def kv_bytes_per_token(self):
        return MLAMemoryManager.bytes_per_token(self.dtype, self.kv_lora, self.rope_d,
                                                self.num_layers + self.extra_kv_layers)

    def _make_mem_manager(self, size):
        if self.extra.get("kv_type") not in (None, "none", "None"):
            raise ValueError("--llm_kv_type: the MLA latent cache has no quantised form here")
        return MLAMemoryManager(size, self.dtype, self.kv_lora, self.rope_d, self.num_layers + self.extra_kv_layers,
                                self.device)

    # ------------------------------------------------------------------ layers
    def _make_decode_state(self, B, b_req_idx, b_seq_len, mem_index, max_kv_len, num_splits=None):
        st = super()._make_decode_state(B, b_req_idx, b_seq_len, mem_index, max_kv_len, num_splits=1)
        dev = self.device
        st.cu_q = torch.arange(B + 1, dtype=torch.int32, device=dev)
        st.b_ready_cache_len = b_seq_len - 1
        return st

    def _attention_block(self, i, lw, h, st):
        T = h.shape[0]
        hq, nope, rope, kvl = self.hq, self.nope, self.rope_d, self.kv_lora
        if self.q_lora:
            qkv_a = ops.gemm(h, lw.qkv_a_w)                       # [T, q_lora + kv_lora + rope]
            q_a = ops.rmsnorm(qkv_a[:, : self.q_lora], lw.q_a_norm, self.eps)
            kv_a = qkv_a[:, self.q_lora:]
            q = ops.gemm(q_a, lw.q_b_w)                           # [T, hq * (nope + rope)]
        else:
            q = ops.gemm(h, lw.q_b_w)
            kv_a = ops.gemm(h, lw.kv_a_w)
        q3 = q.view(T, hq, nope + rope)
        kv_layer = self._kv_layer(i)                      # [slots, 1, kvl + rope]
        ops.mla_rope_kv_scatter_(q3, kv_a, kv_layer, lw.kv_a_norm, self.cos, self.sin, st.position_ids, st.mem_index,
                                 nope, rope, kvl, self.eps)
        q_lat = mla_ops.gemm_batched(q3[:, :, :nope], lw.w_uk)    # [T, hq, kvl]
        o_lat = self._mla_attend(i, lw, h, q_a if self.q_lora else None, q_lat, q3[:, :, nope:], kv_layer, st)
        o = mla_ops.gemm_batched(o_lat, lw.w_uv)                  # [T, hq, v]
        return o.reshape(T, hq * self.v_dim)

    def _mla_attend(self, i, lw, h, q_a, q_lat, q_pe, kv_layer, st):
        """Absorbed attention over the latent cache: [T, hq, kv_lora].  Sparse variants override this."""
        return mla_ops.mla_attention(q_lat, q_pe, kv_layer, self.req_manager.req_to_token_indexs,
                                     st.b_req_idx, st.b_seq_len, st.cu_q, st.b_ready_cache_len, self.kv_lora,
                                     self.sm_scale, st.is_prefill, st.max_q_len, st.max_kv_len,
                                     batch_of=st.batch_of_token if st.is_prefill else None)

    def _ffn_block(self, i, lw, h, st):
        if lw.is_moe:
            return "partial", moe.moe_ffn(self, lw, h, self.moe, layer=i, st=st)
        return self._dense_ffn(lw, h)
