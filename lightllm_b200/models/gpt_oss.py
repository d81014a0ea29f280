"""GPT-OSS: grouped-query attention with a learned sink logit per head, sliding windows on every other layer,
biases on q/k/v/o, YaRN rotary scaling; MoE with a biased router (softmax over the chosen logits), biased
experts and the clamped SwiGLU `(up + 1) * gate * sigmoid(1.702 * gate)`.

Attention runs on the generic paged kernel (it implements sinks and windows); the experts use the grouped
tcgen05 GEMMs with the bias / activation kernels of `csrc/moe.cu`.  The checkpoint stores the expert matrices
transposed ([E, H, 2I] with gate / up columns alternating, [E, I, H]); they are re-laid out at load.
Reference: lightllm/models/gpt_oss.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import moe as moe_ops
from ..ops import reference as ref
from .base import TransformerLM
from .registry import register_model
from .weights import tp_range


@register_model("gpt_oss")
class GptOssLM(TransformerLM):
    model_type = "gpt_oss"

    def _read_config(self, c):
        super()._read_config(c)
        self.attn_bias = True
        self.num_experts = c.get("num_local_experts", c.get("num_experts"))
        self.top_k = c.get("num_experts_per_tok", c.get("experts_per_token", 4))
        w = int(c.get("sliding_window") or 0)
        types = c.get("layer_types") or ["sliding_attention" if i % 2 == 0 else "full_attention"
                                         for i in range(self.num_layers)]
        self.windows = [w if t == "sliding_attention" else 0 for t in types]
        self.ep = bool(self.extra.get("enable_ep_moe", False))

    # ---- weights ----
    def _attn_weight_shapes(self, p):
        s = super()._attn_weight_shapes(p)
        s[p + "self_attn.o_proj.bias"] = (self.hidden,)
        s[p + "self_attn.sinks"] = (self.num_q_heads,)
        return s

    def _ffn_weight_shapes(self, p, layer):
        E, H, I = self.num_experts, self.hidden, self.inter
        return {p + "mlp.router.weight": (E, H), p + "mlp.router.bias": (E,),
                p + "mlp.experts.gate_up_proj": (E, H, 2 * I), p + "mlp.experts.gate_up_proj_bias": (E, 2 * I),
                p + "mlp.experts.down_proj": (E, I, H), p + "mlp.experts.down_proj_bias": (E, H)}

    def _load_attn(self, lw, src, p, layer):
        super()._load_attn(lw, src, p, layer)
        h0, h1 = tp_range(self.num_q_heads, self.tp.rank, self.tp.size)
        lw.sinks = src.get(p + "self_attn.sinks").to(self.device, torch.float32)[h0:h1].contiguous()

    def _load_ffn(self, lw, src, p, layer):
        tp, r = self.tp.size, self.tp.rank
        E, I = self.num_experts, self.inter
        lw.router_w = self._dev(src.get(p + "mlp.router.weight"))
        lw.router_b = self._dev(src.get(p + "mlp.router.bias"))
        if self.ep and tp > 1:
            e0, e1 = tp_range(E, r, tp)
            i0, i1 = 0, I
        else:
            e0, e1 = 0, E
            i0, i1 = tp_range(I, r, tp)
        gu = src.get(p + "mlp.experts.gate_up_proj")[e0:e1]          # [E, H, 2I], columns g0 u0 g1 u1 ...
        gub = src.get(p + "mlp.experts.gate_up_proj_bias")[e0:e1]    # [E, 2I]
        dn = src.get(p + "mlp.experts.down_proj")[e0:e1]             # [E, I, H]
        dnb = src.get(p + "mlp.experts.down_proj_bias")[e0:e1]       # [E, H]
        w13, b13 = [], []
        for e in range(e1 - e0):
            g, u = gu[e][:, 0::2].t()[i0:i1], gu[e][:, 1::2].t()[i0:i1]            # [I_local, H] each
            w13.append(ref.interleave_gate_up(g.contiguous(), u.contiguous()))
            bg, bu = gub[e][0::2][i0:i1], gub[e][1::2][i0:i1]
            b13.append(ref.interleave_gate_up(bg.reshape(-1, 1).contiguous(), bu.reshape(-1, 1).contiguous()).reshape(-1))
        lw.w13 = self._dev(torch.stack(w13))
        lw.b13 = self._dev(torch.stack(b13))
        lw.w2 = self._dev(dn.transpose(1, 2)[:, :, i0:i1])            # [E, H, I_local]
        # the down bias is added once per expert output: with the intermediate dim split over ranks each adds 1/tp
        lw.b2 = self._dev(dnb / (1 if (self.ep and tp > 1) else tp))
        lw.e0 = e0 if (self.ep and tp > 1) else 0

    # ---- layers ----
    def _attention_block(self, i, lw, h, st):
        D, hq, hkv = self.head_dim, self.hq, self.hkv
        qkv = ops.gemm(h, lw.qkv_w, bias=lw.qkv_b)
        kv_layer = self._kv_layer(i)
        ops.rope_kv_scatter_(qkv, kv_layer, self.cos, self.sin, st.position_ids, st.mem_index, hq, hkv, D, self.rot_dim)
        o = ops.attention_generic(qkv[:, : hq * D], kv_layer, self.req_manager.req_to_token_indexs, st.b_req_idx,
                                  st.seq_pos, st.batch_of_token if st.is_prefill else None, hq, hkv, D, self.sm_scale,
                                  window=self.windows[i], sinks=lw.sinks)
        return o.view(-1, hq * D)

    def _ffn_block(self, i, lw, h, st):
        logits = ops.gemm(h, lw.router_w, bias=lw.router_b, epi="f32")
        ids, w = moe_ops.topk_softmax(logits, self.top_k, True, 1.0)
        out = self._partial_out(h.shape[0])
        moe_ops.fused_experts(h, lw.w13, lw.w2, ids, w, "swiglu_oai", lw.e0, out=out, b13=lw.b13, b2=lw.b2)
        return "partial", out
