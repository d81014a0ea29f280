"""Qwen3-Next: a hybrid decoder.  Three of every four layers are Gated DeltaNet linear attention (a per-head matrix
state and a short causal convolution instead of a KV cache), the fourth is softmax attention with an output gate
(q_proj emits query and gate per head), partial rotary embedding (a quarter of the head) and zero-centred RMSNorm
weights (1 + w) everywhere except the gated norm inside the linear layers.  Every layer's FFN is a sparse MoE with one
shared expert scaled by a sigmoid gate.

State: KV pool rows only for the softmax layers; the linear layers keep, per request slot, the last kernel-1 inputs
of the convolution and the fp32 state matrices.  A request's state is reset by its first prefill chunk and carried
over later chunks and decode steps, so prompts cannot share cached prefixes (the prefix cache is switched off for
this family).

Reference: lightllm/models/qwen3next/ (model.py, layer_infer/transformer_layer_infer.py, mem_manager.py,
ReqManagerForMamba in lightllm/common/req_manager.py).
"""
from __future__ import annotations

import re

import torch

from .. import ops
from ..ops import linear_attn as la
from . import moe
from .qwen3_moe import Qwen3MoeLM
from .registry import register_model
from .remap import FusedExperts, RemapSource
from .weights import kv_head_range, tp_range


@register_model("qwen3_next")
class Qwen3NextLM(Qwen3MoeLM):
    model_type = "qwen3_next"
    # a shared prefix is usable only with the linear layers' state at its end: `engine/state_cache.py` keeps
    # snapshots at page boundaries when the model is built with state_snapshot_slots > 0
    supports_prefix_cache = False

    # ------------------------------------------------------------------ config
    def _read_config(self, c):
        c = dict(c)
        c.setdefault("partial_rotary_factor", (c.get("rope_parameters") or {}).get("partial_rotary_factor", 0.25))
        super()._read_config(c)
        self.norm_w_offset = 1.0
        n = self.num_layers
        interval = int(c.get("full_attention_interval", 4))
        self.layer_types = list(c.get("layer_types") or
                                ["full_attention" if (i + 1) % interval == 0 else "linear_attention" for i in range(n)])
        self.full_layers = [i for i, t in enumerate(self.layer_types) if t == "full_attention"]
        self.lin_layers = [i for i, t in enumerate(self.layer_types) if t != "full_attention"]
        self._kv_slot = {i: j for j, i in enumerate(self.full_layers)}
        self._lin_slot = {i: j for j, i in enumerate(self.lin_layers)}
        self.nk_all, self.nv_all = c["linear_num_key_heads"], c["linear_num_value_heads"]
        self.dk, self.dv = c["linear_key_head_dim"], c["linear_value_head_dim"]
        self.conv_k = int(c.get("linear_conv_kernel_dim", 4))
        tp, r = self.tp.size, self.tp.rank
        assert self.nk_all % tp == 0, "linear key heads must divide by tp"
        self._nk_range = tp_range(self.nk_all, r, tp)
        self.nk = self._nk_range[1] - self._nk_range[0]
        self.vrep = self.nv_all // self.nk_all
        self.nv = self.nk * self.vrep
        self.conv_dim = 2 * self.nk * self.dk + self.nv * self.dv
        self.moe = moe.MoEConfig(c["num_experts"], c["num_experts_per_tok"], c["moe_intermediate_size"],
                                 renorm=c.get("norm_topk_prob", True), act=self.act,
                                 n_shared=1 if c.get("shared_expert_intermediate_size") else 0,
                                 shared_inter=c.get("shared_expert_intermediate_size") or 0,
                                 shared_name="shared_expert", shared_gate=True)

    # ------------------------------------------------------------------ weights
    def _wrap_source(self, src):
        """Checkpoints that store a layer's experts as two 3-D tensors are presented per expert."""
        fused = [n for n in src.names() if n.endswith("mlp.experts.gate_up_proj")]
        if not fused:
            return src
        t = {n: n for n in src.names()}
        I, H, cache = self.moe.inter, self.hidden, FusedExperts()
        for n in fused:
            p = n[: -len("gate_up_proj")]
            for e in range(self.moe.num_experts):
                t[f"{p}{e}.gate_proj.weight"] = cache.entry(n, e, 2 * I, 0, I)
                t[f"{p}{e}.up_proj.weight"] = cache.entry(n, e, 2 * I, I, 2 * I)
                t[f"{p}{e}.down_proj.weight"] = cache.entry(p + "down_proj", e, H)
            t.pop(n)
            t.pop(p + "down_proj", None)
        return RemapSource(src, t)

    def _attn_weight_shapes(self, p):
        i = int(re.search(r"layers\.(\d+)\.", p).group(1))
        H, D = self.hidden, self.head_dim
        if self.layer_types[i] == "full_attention":
            return {p + "self_attn.q_proj.weight": (self.num_q_heads * D * 2, H),
                    p + "self_attn.k_proj.weight": (self.num_kv_heads * D, H),
                    p + "self_attn.v_proj.weight": (self.num_kv_heads * D, H),
                    p + "self_attn.o_proj.weight": (H, self.num_q_heads * D),
                    p + "self_attn.q_norm.weight": (D,), p + "self_attn.k_norm.weight": (D,)}
        kd, vd = self.nk_all * self.dk, self.nv_all * self.dv
        a = p + "linear_attn."
        return {a + "in_proj_qkvz.weight": (2 * kd + 2 * vd, H), a + "in_proj_ba.weight": (2 * self.nv_all, H),
                a + "conv1d.weight": (2 * kd + vd, 1, self.conv_k), a + "dt_bias": (self.nv_all,),
                a + "A_log": (self.nv_all,), a + "norm.weight": (self.dv,), a + "out_proj.weight": (H, vd)}

    def _load_attn(self, lw, src, p, layer):
        H, D = self.hidden, self.head_dim
        tp, r = self.tp.size, self.tp.rank
        if self.layer_types[layer] == "full_attention":
            q0, q1 = tp_range(self.num_q_heads, r, tp)
            k0, k1 = self._kv_range
            qg = src.get(p + "self_attn.q_proj.weight", 0, q0 * 2 * D, q1 * 2 * D).view(q1 - q0, 2, D, H)
            k = src.get(p + "self_attn.k_proj.weight", 0, k0 * D, k1 * D)
            v = src.get(p + "self_attn.v_proj.weight", 0, k0 * D, k1 * D)
            # one GEMM gives [q | k | v | gate]: the first three are what the attention path expects
            lw.qkv_w = self._dev(torch.cat([qg[:, 0].reshape(-1, H), k, v, qg[:, 1].reshape(-1, H)], dim=0))
            lw.o_w = self._dev(src.get(p + "self_attn.o_proj.weight", 1, q0 * D, q1 * D))
            lw.q_norm = self._dev(src.get(p + "self_attn.q_norm.weight"))
            lw.k_norm = self._dev(src.get(p + "self_attn.k_norm.weight"))
            lw.is_linear = False
            return
        a = p + "linear_attn."
        n0, n1 = self._nk_range
        per_k = 2 * self.dk + 2 * self.vrep * self.dv          # rows of in_proj_qkvz per key head: [q | k | v | z]
        qkvz = src.get(a + "in_proj_qkvz.weight", 0, n0 * per_k, n1 * per_k)
        ba = src.get(a + "in_proj_ba.weight", 0, n0 * 2 * self.vrep, n1 * 2 * self.vrep)
        lw.in_w = self._dev(torch.cat([qkvz, ba], dim=0))
        conv = src.get(a + "conv1d.weight").reshape(-1, self.conv_k)
        kd_all = self.nk_all * self.dk
        parts = [conv[n0 * self.dk:n1 * self.dk], conv[kd_all + n0 * self.dk:kd_all + n1 * self.dk],
                 conv[2 * kd_all + n0 * self.vrep * self.dv:2 * kd_all + n1 * self.vrep * self.dv]]
        lw.conv_w = torch.cat(parts, dim=0).to(self.device, torch.float32).contiguous()
        v0, v1 = n0 * self.vrep, n1 * self.vrep
        lw.neg_a = (-src.get(a + "A_log").float().exp())[v0:v1].to(self.device).contiguous()
        lw.dt_bias = src.get(a + "dt_bias").float()[v0:v1].to(self.device).contiguous()
        lw.gnorm_w = src.get(a + "norm.weight").to(self.device, torch.float32).contiguous()
        lw.o_w = self._dev(src.get(a + "out_proj.weight", 1, v0 * self.dv, v1 * self.dv))
        lw.is_linear = True

    # ------------------------------------------------------------------ memory
    def kv_bytes_per_token(self):
        return self._kv_manager_class().bytes_per_token(self.dtype, self.hkv, self.head_dim,
                                                        len(self.full_layers) + self.extra_kv_layers)

    def _make_mem_manager(self, size):
        return self._kv_manager_class()(size, self.dtype, self.hkv, self.head_dim,
                                        len(self.full_layers) + self.extra_kv_layers, self.device,
                                        **self._kv_manager_kwargs())

    def _kv_layer(self, i: int):
        return self.mem_manager.layer(self.kv_layer_offset + self._kv_slot[i])

    def _init_mem(self, max_total_token_num, mem_fraction):
        # the per-request state of the linear layers comes out of the same budget: allocate it first
        rows = self.max_req_num + 1
        n = len(self.lin_layers)
        self.conv_state = torch.zeros((n, rows, self.conv_dim, self.conv_k - 1), dtype=self.dtype, device=self.device)
        # `--linear_att_ssm_data_type bfloat16` halves the recurrent state (updates still run in fp32)
        ssm_dtype = torch.bfloat16 if str(self.extra.get("linear_att_ssm_data_type", "float32")) in ("bfloat16", "bf16") \
            else torch.float32
        self.ssm_state = torch.zeros((n, rows, self.nv, self.dk, self.dv), dtype=ssm_dtype, device=self.device)
        self._verify_snaps = {}
        self.state_snapshot_slots = int(self.extra.get("state_snapshot_slots") or 0)
        if self.state_snapshot_slots > 0:
            k = self.state_snapshot_slots
            self.conv_snap = torch.zeros((k, n, self.conv_dim, self.conv_k - 1), dtype=self.dtype, device=self.device)
            self.ssm_snap = torch.zeros((k, n, self.nv, self.dk, self.dv), dtype=ssm_dtype, device=self.device)
        super()._init_mem(max_total_token_num, mem_fraction)

    needs_state_rollback = True   # a verification pass must be followed by `commit_verify`

    def save_state_snapshot(self, slot: int, req_idx: int):
        self.conv_snap[slot].copy_(self.conv_state[:, req_idx])
        self.ssm_snap[slot].copy_(self.ssm_state[:, req_idx])

    def load_state_snapshot(self, slot: int, req_idx: int):
        self.conv_state[:, req_idx] = self.conv_snap[slot]
        self.ssm_state[:, req_idx] = self.ssm_snap[slot]

    # host tier of the snapshot table (engine/state_cache.py)
    def alloc_host_snapshots(self, nbytes: int) -> int:
        """Pinned host room for as many snapshots as fit into `nbytes`; returns their number."""
        one = self.conv_snap[0].numel() * self.conv_snap.element_size() + \
            self.ssm_snap[0].numel() * self.ssm_snap.element_size()
        k = int(nbytes) // max(one, 1)
        if k <= 0:
            return 0
        pin = self.device.type == "cuda"
        self.conv_host = torch.empty((k, *self.conv_snap.shape[1:]), dtype=self.conv_snap.dtype, pin_memory=pin)
        self.ssm_host = torch.empty((k, *self.ssm_snap.shape[1:]), dtype=self.ssm_snap.dtype, pin_memory=pin)
        return k

    def export_state_snapshot(self, slot: int, host_slot: int):
        self.conv_host[host_slot].copy_(self.conv_snap[slot])      # synchronous: the GPU slot is reused right after
        self.ssm_host[host_slot].copy_(self.ssm_snap[slot])

    def import_state_snapshot(self, host_slot: int, slot: int):
        self.conv_snap[slot].copy_(self.conv_host[host_slot], non_blocking=True)
        self.ssm_snap[slot].copy_(self.ssm_host[host_slot], non_blocking=True)

    def commit_verify(self, n_keep):
        """After a verification pass (`verify_pass=True`) over the batch: request b keeps its first n_keep[b] >= 1
        positions; the recurrent state of every linear layer is set to the state after that position."""
        n_keep = torch.as_tensor(n_keep, dtype=torch.long, device=self.device)
        for slot, (req, conv_snaps, ssm_snaps) in self._verify_snaps.items():
            b = torch.arange(req.shape[0], device=self.device)
            self.conv_state[slot].index_copy_(0, req, conv_snaps[b, n_keep - 1])
            self.ssm_state[slot].index_copy_(0, req, ssm_snaps[b, n_keep - 1].to(self.ssm_state.dtype))
        self._verify_snaps.clear()

    # ------------------------------------------------------------------ layers
    def _attention_block(self, i, lw, h, st):
        if lw.is_linear:
            return self._linear_attention(i, lw, h, st)
        D, hq, hkv = self.head_dim, self.hq, self.hkv
        qkvg = ops.gemm(h, lw.qkv_w)
        n_qkv = (hq + 2 * hkv) * D
        qkv, gate = qkvg[:, :n_qkv], qkvg[:, n_qkv:]
        kv_layer = self._kv_layer(i)
        cos, sin, rope_rows = self._rope_inputs(st, i)
        ops.rope_kv_scatter_(qkv, kv_layer, cos, sin, rope_rows, st.mem_index, hq, hkv, D, self.rot_dim, lw.q_norm,
                             lw.k_norm, self.eps, self.norm_w_offset)
        q = qkv[:, : hq * D]
        r2t = self.req_manager.req_to_token_indexs
        if D not in (64, 128):
            o = ops.attention_generic(q, kv_layer, r2t, st.b_req_idx, st.seq_pos,
                                      st.batch_of_token if st.is_prefill else None, hq, hkv, D, self.sm_scale)
        elif st.is_prefill:
            o = ops.gqa_prefill(q, kv_layer, r2t, st.b_req_idx, st.cu_q, st.b_ready_cache_len, hq, hkv, D,
                                st.max_q_len, self.sm_scale)
        else:
            o = ops.gqa_decode(q, kv_layer, r2t, st.b_req_idx, st.b_seq_len, hq, hkv, D, st.max_kv_len, self.sm_scale,
                               num_splits=st.decode_num_splits, scratch=st.decode_scratch)
        o = o.reshape(-1, hq * D)
        return (o.float() * torch.sigmoid(gate.float())).to(o.dtype)

    def _split_projection(self, proj):
        """[T, P] -> q, k [T, nk, dk], v, z [T, nv, dv], b, a [T, nv]."""
        T = proj.shape[0]
        per_k = 2 * self.dk + 2 * self.vrep * self.dv
        nq = self.nk * per_k
        qkvz = proj[:, :nq].view(T, self.nk, per_k)
        ba = proj[:, nq:].view(T, self.nk, 2 * self.vrep)
        q, k = qkvz[..., : self.dk], qkvz[..., self.dk:2 * self.dk]
        v = qkvz[..., 2 * self.dk:2 * self.dk + self.vrep * self.dv].reshape(T, self.nv, self.dv)
        z = qkvz[..., 2 * self.dk + self.vrep * self.dv:].reshape(T, self.nv, self.dv)
        b, a = ba[..., : self.vrep].reshape(T, self.nv), ba[..., self.vrep:].reshape(T, self.nv)
        return q, k, v, z, b, a

    def _linear_attention(self, i, lw, h, st):
        T = h.shape[0]
        slot = self._lin_slot[i]
        q, k, v, z, b, a = self._split_projection(ops.gemm(h, lw.in_w))
        kd = self.nk * self.dk
        mixed = torch.cat([q.reshape(T, kd), k.reshape(T, kd), v.reshape(T, self.nv * self.dv)], dim=1).float()
        beta = torch.sigmoid(b.float())
        g = lw.neg_a * torch.nn.functional.softplus(a.float() + lw.dt_bias)
        conv_state, ssm_state = self.conv_state[slot], self.ssm_state[slot]

        def heads(m):
            qq = m[:, :kd].view(-1, self.nk, self.dk).repeat_interleave(self.vrep, dim=1)
            kk = m[:, kd:2 * kd].view(-1, self.nk, self.dk).repeat_interleave(self.vrep, dim=1)
            return qq, kk, m[:, 2 * kd:].view(-1, self.nv, self.dv)

        if not st.is_prefill and h.is_cuda and la.step_kernel_supported(self.dk, self.dv, self.conv_k):
            # one token per request: convolution step + state update / read-out, two kernels
            core = la.conv_and_delta_step(mixed.contiguous(), conv_state, lw.conv_w, ssm_state,
                                          st.b_req_idx.to(torch.int32), g.float(), beta, self.nk, self.nv, self.dk,
                                          self.dv)
        elif not st.is_prefill:  # one token per request, all requests at once (torch restatement)
            req = st.b_req_idx.long()
            y, new_conv = la.causal_conv_step(mixed, conv_state[req], lw.conv_w)
            conv_state.index_copy_(0, req, new_conv.to(conv_state.dtype))
            qq, kk, vv = heads(y)
            core, new_s = la.gated_delta_step(qq, kk, vv, g, beta, ssm_state[req])
            ssm_state.index_copy_(0, req, new_s.to(ssm_state.dtype))
        elif st.extra.get("verify_pass"):
            # speculative verification: every request brings the same number of tokens; they go through the
            # recurrence one position at a time and the state after every position is kept, so that
            # `commit_verify` can restore the state at the last accepted position
            req = st.b_req_idx.long()
            B = req.shape[0]
            qn = T // B
            cs, ss = conv_state[req], ssm_state[req].float()
            conv_snaps, ssm_snaps, cores = [], [], []
            for t in range(qn):
                y, cs = la.causal_conv_step(mixed[t::qn], cs, lw.conv_w)
                cs = cs.to(conv_state.dtype)
                qq, kk, vv = heads(y)
                o, ss = la.gated_delta_step(qq, kk, vv, g[t::qn], beta[t::qn], ss)
                conv_snaps.append(cs)
                ssm_snaps.append(ss)
                cores.append(o)
            self._verify_snaps[slot] = (req, torch.stack(conv_snaps, dim=1), torch.stack(ssm_snaps, dim=1))
            conv_state.index_copy_(0, req, cs)
            ssm_state.index_copy_(0, req, ss.to(ssm_state.dtype))
            core = torch.stack(cores, dim=1).reshape(T, self.nv, self.dv)
        else:
            q_len, ready, reqs = st.extra["q_len_cpu"].tolist(), st.extra["ready_cpu"].tolist(), \
                st.extra["req_idx_cpu"].tolist()
            outs, off = [], 0
            for n, r, rq in zip(q_len, ready, reqs):
                if r == 0:  # first chunk of this request: fresh state
                    conv_state[rq].zero_()
                    ssm_state[rq].zero_()
                y, new_conv = la.causal_conv_prefill(mixed[off:off + n], conv_state[rq], lw.conv_w)
                conv_state[rq].copy_(new_conv)
                qq, kk, vv = heads(y)
                o, new_s = la.gated_delta_chunked(qq, kk, vv, g[off:off + n], beta[off:off + n], ssm_state[rq])
                ssm_state[rq].copy_(new_s)
                outs.append(o)
                off += n
            core = torch.cat(outs, dim=0)
        out = la.rmsnorm_gated(core, z, lw.gnorm_w, self.eps)
        return out.reshape(T, self.nv * self.dv).to(h.dtype)


class _SeparateProjections:
    """Qwen3.5 stores the linear layers' input projections as four matrices (`in_proj_qkv` with all q heads, then
    all k heads, then all v heads; `in_proj_z`, `in_proj_b`, `in_proj_a`): they are regrouped per key head at load
    into the layout `_split_projection` reads."""

    def _attn_weight_shapes(self, p):
        s = super()._attn_weight_shapes(p)
        a = p + "linear_attn."
        if a + "in_proj_qkvz.weight" in s:
            H = self.hidden
            kd, vd = self.nk_all * self.dk, self.nv_all * self.dv
            s.pop(a + "in_proj_qkvz.weight")
            s.pop(a + "in_proj_ba.weight")
            s.update({a + "in_proj_qkv.weight": (2 * kd + vd, H), a + "in_proj_z.weight": (vd, H),
                      a + "in_proj_b.weight": (self.nv_all, H), a + "in_proj_a.weight": (self.nv_all, H)})
        return s

    def _load_attn(self, lw, src, p, layer):
        if self.layer_types[layer] == "full_attention":
            return super()._load_attn(lw, src, p, layer)
        a = p + "linear_attn."
        n0, n1 = self._nk_range
        H, dk, dv, r = self.hidden, self.dk, self.dv, self.vrep
        kd_all = self.nk_all * dk
        qkv = src.get(a + "in_proj_qkv.weight")
        q = qkv[n0 * dk:n1 * dk].view(self.nk, dk, H)
        k = qkv[kd_all + n0 * dk:kd_all + n1 * dk].view(self.nk, dk, H)
        v = qkv[2 * kd_all + n0 * r * dv:2 * kd_all + n1 * r * dv].view(self.nk, r * dv, H)
        z = src.get(a + "in_proj_z.weight", 0, n0 * r * dv, n1 * r * dv).view(self.nk, r * dv, H)
        b = src.get(a + "in_proj_b.weight", 0, n0 * r, n1 * r).view(self.nk, r, H)
        aa = src.get(a + "in_proj_a.weight", 0, n0 * r, n1 * r).view(self.nk, r, H)
        grouped = torch.cat([q, k, v, z], dim=1).reshape(-1, H)
        ba = torch.cat([b, aa], dim=1).reshape(-1, H)

        class _View:  # the grouped matrices under the names the parent loader asks for
            def __init__(self, base):
                self.base = base

            def get(self, name, dim=None, start=0, end=None):
                if name == a + "in_proj_qkvz.weight":
                    return grouped
                if name == a + "in_proj_ba.weight":
                    return ba
                return self.base.get(name, dim, start, end)

            def has(self, name):
                return self.base.has(name)

        self._load_linear_from(lw, _View(src), p, (n0, n1))


def _load_linear_from(self, lw, src, p, real_range):
    """The linear layer's tensors with the input projections taken whole from `src` (already this rank's heads,
    grouped per key head) and every other per-head tensor sliced by the rank's head range."""
    a = p + "linear_attn."
    n0, n1 = real_range
    per_k = 2 * self.dk + 2 * self.vrep * self.dv
    lw.in_w = self._dev(torch.cat([src.get(a + "in_proj_qkvz.weight")[: self.nk * per_k],
                                   src.get(a + "in_proj_ba.weight")], dim=0))
    conv = src.get(a + "conv1d.weight").reshape(-1, self.conv_k)
    kd_all = self.nk_all * self.dk
    parts = [conv[n0 * self.dk:n1 * self.dk], conv[kd_all + n0 * self.dk:kd_all + n1 * self.dk],
             conv[2 * kd_all + n0 * self.vrep * self.dv:2 * kd_all + n1 * self.vrep * self.dv]]
    lw.conv_w = torch.cat(parts, dim=0).to(self.device, torch.float32).contiguous()
    v0, v1 = n0 * self.vrep, n1 * self.vrep
    lw.neg_a = (-src.get(a + "A_log").float().exp())[v0:v1].to(self.device).contiguous()
    lw.dt_bias = src.get(a + "dt_bias").float()[v0:v1].to(self.device).contiguous()
    lw.gnorm_w = src.get(a + "norm.weight").to(self.device, torch.float32).contiguous()
    lw.o_w = self._dev(src.get(a + "out_proj.weight", 1, v0 * self.dv, v1 * self.dv))
    lw.is_linear = True


_SeparateProjections._load_linear_from = _load_linear_from


def _strip_language_model_prefix(src):
    for pre in ("model.language_model.", "language_model.model."):
        if src.has(pre + "embed_tokens.weight"):
            return RemapSource(src, {"model." + n[len(pre):]: n for n in src.names() if n.startswith(pre)})
    return src


@register_model("qwen3_5_moe", "qwen3_5_moe_text")
class Qwen3_5MoeLM(_SeparateProjections, Qwen3NextLM):
    """Qwen3.5-MoE language model (text path): the Qwen3-Next layer stack with separately stored input projections.
    Reference: lightllm/models/qwen3_5_moe/."""

    model_type = "qwen3_5_moe"

    def _wrap_source(self, src):
        return super()._wrap_source(_strip_language_model_prefix(src))


@register_model("qwen3_5", "qwen3_5_text")
class Qwen3_5LM(_SeparateProjections, Qwen3NextLM):
    """Qwen3.5 dense language model (text path): hybrid attention as Qwen3-Next, plain SwiGLU FFN in every layer.
    Reference: lightllm/models/qwen3_5/."""

    model_type = "qwen3_5"

    def _read_config(self, c):
        c = dict(c)
        c.setdefault("num_experts", 1)
        c.setdefault("num_experts_per_tok", 1)
        c.setdefault("moe_intermediate_size", c.get("intermediate_size"))
        super()._read_config(c)
        self._moe_layers = set()  # every FFN is dense
        self.moe = None

    def _wrap_source(self, src):
        return _strip_language_model_prefix(src)
