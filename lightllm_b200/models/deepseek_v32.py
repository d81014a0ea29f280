"""DeepSeek-V3.2: the V3 decoder with DeepSeek Sparse Attention.  Every layer carries a small "lightning indexer":
per token it produces `index_n_heads` query vectors (from the q latent) and ONE key vector (LayerNorm of a
projection of the hidden state) of `index_head_dim`, rotary-embedded on their first `qk_rope_head_dim`
dimensions in the half-split layout, and per-head weights; the score of a cached token s for a query token t is

    I[t, s] = sum_h  w[t, h] * relu(q[t, h] . k[s]),      w = weights_proj(x) * index_n_heads^-1/2 * index_head_dim^-1/2

and the absorbed MLA attention of t runs over the `index_topk` best-scoring tokens s <= t only.  The indexer keys
live in a per-layer cache next to the latent KV cache (same slots).

While a batch's contexts are no longer than `index_topk` every token is selected and the dense MLA kernel runs.
Beyond that the scores and the selection run on torch ops (stable sort) and the attention over the selected tokens is
one launch of the MLA kernel in its decode form over per-token slot lists (`_sparse_attend`), outside CUDA graphs.
The reference quantises the indexer's q and k to fp8
after a Hadamard rotation (which leaves q . k unchanged); here they stay in the compute dtype.

Reference: lightllm/models/deepseek3_2/{model.py,layer_infer/transformer_layer_infer.py (NsaInfer),
layer_weights/transformer_layer_weight.py}, common/basemodel/attention/nsa/*.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import ops
from ..ops import mla as mla_ops
from .deepseek2 import DeepseekV2LM
from .registry import register_model


@register_model("deepseek_v32")
class DeepseekV32LM(DeepseekV2LM):
    model_type = "deepseek_v32"

    def _read_config(self, c):
        super()._read_config(c)
        assert self.q_lora, "the indexer reads the q latent"
        self.idx_heads = int(c["index_n_heads"])
        self.idx_dim = int(c["index_head_dim"])
        self.idx_topk = int(c["index_topk"])
        self.idx_scale = self.idx_heads ** -0.5 * self.idx_dim ** -0.5

    # ------------------------------------------------------------------ weights
    def _attn_weight_shapes(self, p):
        s = super()._attn_weight_shapes(p)
        a = p + "self_attn.indexer."
        s.update({a + "wq_b.weight": (self.idx_heads * self.idx_dim, self.q_lora), a + "wk.weight": (self.idx_dim, self.hidden),
                  a + "k_norm.weight": (self.idx_dim,), a + "k_norm.bias": (self.idx_dim,),
                  a + "weights_proj.weight": (self.idx_heads, self.hidden)})
        return s

    def fp8_weight_names(self):
        return {n for n in super().fp8_weight_names() if "indexer." not in n}

    def weight_shapes(self):
        return {n: shp for n, shp in super().weight_shapes().items()
                if not ("indexer." in n and n.endswith("_scale_inv"))}

    def _load_attn(self, lw, src, p, layer):
        super()._load_attn(lw, src, p, layer)
        a = p + "self_attn.indexer."
        # the indexer is small: every rank keeps all of its heads, so the selection needs no communication
        lw.idx_wq = self._dev(self._w(src, a + "wq_b.weight"))
        lw.idx_wk = self._dev(self._w(src, a + "wk.weight"))
        lw.idx_kn_w = src.get(a + "k_norm.weight").to(self.device, torch.float32)
        lw.idx_kn_b = src.get(a + "k_norm.bias").to(self.device, torch.float32)
        lw.idx_wp = self._dev(self._w(src, a + "weights_proj.weight"))

    # ------------------------------------------------------------------ memory
    def kv_bytes_per_token(self):
        n = self.num_layers + self.extra_kv_layers
        return super().kv_bytes_per_token() + n * self.idx_dim * torch.empty((), dtype=self.dtype).element_size()

    def _init_mem(self, max_total_token_num, mem_fraction):
        super()._init_mem(max_total_token_num, mem_fraction)
        if not self.disable_cudagraph and self.graph_max_len_in_batch > self.idx_topk:
            # contexts beyond index_topk take the selection path, whose shapes depend on the batch
            self.graph_max_len_in_batch = self.idx_topk
        if self.share_with is None:
            n = self.num_layers + self.extra_kv_layers
            self.index_k = torch.zeros((n, self.mem_manager.size + 1, self.idx_dim), dtype=self.dtype,
                                       device=self.device)
        else:
            self.index_k = self.share_with.index_k

    # ------------------------------------------------------------------ attention
    def _rope_half(self, x, pos):
        """Half-split rotary embedding on the first `rope_d` dimensions of the last axis (fp32 in, fp32 out)."""
        R = self.rope_d
        cos, sin = self.cos[pos].float(), self.sin[pos].float()            # [T, R / 2]
        while cos.dim() < x.dim():
            cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
        x1, x2 = x[..., : R // 2], x[..., R // 2:R]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin, x[..., R:]], dim=-1)

    def _mla_attend(self, i, lw, h, q_a, q_lat, q_pe, kv_layer, st):
        T = h.shape[0]
        Hn, Dn = self.idx_heads, self.idx_dim
        pos = st.position_ids.long()
        ki = F.layer_norm(ops.gemm(h, lw.idx_wk).float(), (Dn,), lw.idx_kn_w, lw.idx_kn_b, self.eps)
        ki = self._rope_half(ki, pos)
        idx_layer = self.index_k[self.kv_layer_offset + i]
        idx_layer[st.mem_index.long()] = ki.to(idx_layer.dtype)
        if st.max_kv_len <= self.idx_topk:                                  # everything is selected
            return super()._mla_attend(i, lw, h, q_a, q_lat, q_pe, kv_layer, st)
        qi = self._rope_half(ops.gemm(q_a, lw.idx_wq).view(T, Hn, Dn).float(), pos)
        w = ops.gemm(h, lw.idx_wp).float() * self.idx_scale                # [T, Hn]
        return self._sparse_attend(qi, w, idx_layer, q_lat, q_pe, kv_layer, st)

    def _sparse_attend(self, qi, w, idx_layer, q_lat, q_pe, kv_layer, st):
        """Index scores of every query token over its request's context, top-k selection under the causal mask, then
        ONE launch of the absorbed-MLA attention kernel in its decode form over per-token slot lists: token t is
        handed to the kernel as a "request" whose table row holds the slots selected for it.  Decode batches are
        scored in one batched product; prompt passes per request (their score matrices differ in shape)."""
        dev = q_lat.device
        r2t = self.req_manager.req_to_token_indexs
        T, K = q_lat.shape[0], self.idx_topk
        B = st.b_req_idx.shape[0]
        sel = torch.zeros((T, K), dtype=torch.int32, device=dev)
        sel_len = torch.empty(T, dtype=torch.int32, device=dev)

        def pick(score, k):
            # stable order: equal scores (e.g. all heads cut off by the relu) keep the earlier token, whatever the
            # shape of the call; masked entries (-inf) sort behind every real one
            return score.sort(dim=-1, descending=True, stable=True).indices[:, :k]

        if not st.is_prefill:
            S = int(st.max_kv_len)
            lens = st.b_seq_len.long()
            rows = r2t.index_select(0, st.b_req_idx.long())[:, :S]                       # [B, S] slots
            kk = idx_layer[rows.long()].float()                                          # [B, S, Dn]
            score = (torch.relu(torch.einsum("bhd,bsd->bhs", qi, kk)) * w.unsqueeze(-1)).sum(1)   # [B, S]
            score = score.masked_fill(torch.arange(S, device=dev)[None, :] >= lens[:, None], float("-inf"))
            k = min(K, S)
            sel[:, :k] = rows.gather(1, pick(score, k))
            sel_len.copy_(lens.clamp(max=K))
        else:
            req_cpu, len_cpu = st.b_req_idx.tolist(), st.b_seq_len.tolist()
            q_len = st.extra["q_len_cpu"].tolist()
            off = 0
            for b in range(B):
                n, S = int(q_len[b]), int(len_cpu[b])
                sl = slice(off, off + n)
                slots = r2t[req_cpu[b], :S]
                qpos = torch.arange(S - n, S, device=dev)                                # positions of the query tokens
                causal = torch.arange(S, device=dev)[None, :] <= qpos[:, None]           # [n, S]
                kk = idx_layer[slots.long()].float()                                     # [S, Dn]
                score = (torch.relu(torch.einsum("thd,sd->ths", qi[sl], kk)) * w[sl].unsqueeze(-1)).sum(1)   # [n, S]
                score = score.masked_fill(~causal, float("-inf"))
                k = min(K, S)
                sel[sl, :k] = slots[pick(score, k)]
                sel_len[sl] = (qpos + 1).clamp(max=K).to(torch.int32)
                off += n
        tok = torch.arange(T + 1, dtype=torch.int32, device=dev)
        return mla_ops.mla_attention(q_lat.contiguous(), q_pe, kv_layer, sel, tok[:T], sel_len, tok, sel_len - 1,
                                     self.kv_lora, self.sm_scale, False, 1, K)
