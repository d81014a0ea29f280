"""Mixture-of-experts FFN shared by the MoE model families.

Expert weights of a layer are two stacked tensors: `w13 [E_local, 2*I_local, H]` (gate and up rows
interleaved in 32-row blocks, so the grouped GEMM's epilogue applies the gated activation) and
`w2 [E_local, H, I_local]`.  Two sharding modes:

  * tensor parallel (default): every rank holds all experts, each sliced along the intermediate
    dimension (I_local = I / tp)
  * expert parallel (`enable_ep_moe`): every rank holds E / tp whole experts (E / world under `--dp`; a replica
    may itself be tensor parallel, its ranks then share the replica's tokens out between them for the exchange).  With tensor-parallel
    attention the hidden states are replicated, so a rank simply evaluates its own experts for all
    tokens (pairs routed elsewhere are dropped by the alignment kernel) -- no all-to-all needed.

Either way the layer produces a per-rank partial sum that goes through the same fused
reduce + residual + RMSNorm as a dense row-parallel GEMM.  With data-parallel attention (`dp == tp`)
tokens differ per rank and `parallel.ep` moves them (dispatch / combine).

Reference: lightllm/common/basemodel/layer_weights/meta_weights/fused_moe/fused_moe_weight.py,
lightllm/common/basemodel/triton_kernel/fused_moe/*, models/qwen3_moe, models/deepseek2 (_moe_ffn*).
"""
from __future__ import annotations

import re

import torch

from .. import ops
from ..ops import moe as moe_ops
from ..ops import reference as ref
from .weights import tp_range


class MoEConfig:
    def __init__(self, num_experts, top_k, inter, renorm=True, scoring="softmax", n_group=1, topk_group=1,
                 routed_scale=1.0, has_bias=False, n_shared=0, shared_inter=0, act="silu",
                 shared_name="shared_experts", shared_gate=False):
        self.num_experts, self.top_k, self.inter = num_experts, top_k, inter
        self.renorm, self.scoring = renorm, scoring
        self.n_group, self.topk_group = n_group, topk_group
        self.routed_scale, self.has_bias = routed_scale, has_bias
        self.n_shared, self.shared_inter = n_shared, shared_inter
        self.act = act
        # checkpoint prefix of the shared expert and whether its output is scaled by sigmoid(x . w_gate)
        # (`shared_expert_gate`, Qwen2-MoE / Qwen3-Next)
        self.shared_name, self.shared_gate = shared_name, shared_gate


def expert_weight_shapes(prefix: str, mc: MoEConfig, hidden: int, gate_name="gate", experts_name="experts"):
    s = {prefix + f"{gate_name}.weight": (mc.num_experts, hidden)}
    if mc.has_bias:
        s[prefix + f"{gate_name}.e_score_correction_bias"] = (mc.num_experts,)
    for e in range(mc.num_experts):
        q = prefix + f"{experts_name}.{e}."
        s[q + "gate_proj.weight"] = (mc.inter, hidden)
        s[q + "up_proj.weight"] = (mc.inter, hidden)
        s[q + "down_proj.weight"] = (hidden, mc.inter)
    if mc.n_shared:
        q = prefix + mc.shared_name + "."
        s[q + "gate_proj.weight"] = (mc.shared_inter, hidden)
        s[q + "up_proj.weight"] = (mc.shared_inter, hidden)
        s[q + "down_proj.weight"] = (hidden, mc.shared_inter)
        if mc.shared_gate:
            s[prefix + mc.shared_name + "_gate.weight"] = (1, hidden)
    return s


def load_experts(model, lw, src, prefix: str, mc: MoEConfig, ep: bool, gate_name="gate", experts_name="experts"):
    """Fills lw.router_w (fp32 logits GEMM runs in bf16 weights), lw.w13, lw.w2, lw.e0, lw.e_local (+ shared expert)."""
    tp, r = model.tp.size, model.tp.rank
    if ep and model.ps.dp_size > 1:  # data-parallel attention: the experts are spread over every rank of the world
        tp, r = model.ps.world_size, model.ps.global_rank
    dev = model._dev
    lw.router_w = dev(src.get(prefix + f"{gate_name}.weight"))
    if mc.has_bias and src.has(prefix + f"{gate_name}.e_score_correction_bias"):
        lw.router_bias = src.get(prefix + f"{gate_name}.e_score_correction_bias").to(model.device, torch.float32)
    if ep and tp > 1:
        e0, e1 = tp_range(mc.num_experts, r, tp)
        i0, i1 = 0, mc.inter
    else:
        e0, e1 = 0, mc.num_experts
        i0, i1 = tp_range(mc.inter, r, tp)
    # redundant experts (data-parallel attention + expert parallelism only): R more slots behind the rank's own experts
    red_ids, layer_no = [], -1
    red_cfg = getattr(model, "redundancy_cfg", None)
    if ep and tp > 1 and model.ps.dp_size > 1 and red_cfg is not None and red_cfg.num > 0:
        m = re.search(r"layers\.(\d+)\.", prefix)
        layer_no = int(m.group(1)) if m else -1
        red_ids = red_cfg.ids(layer_no)
    expert_ids = list(range(e0, e1)) + red_ids
    raw = getattr(src, "base", src)  # the fp8 payload lives under a de-quantising view
    use_fp8 = getattr(model, "fp8_compute", False) and i0 % 128 == 0 and (i1 - i0) % 128 == 0 and mc.act == "silu"

    def read_expert(e: int):
        """(w13, w2) of one expert as they are stacked: host tensors (bf16) or one-expert Fp8Weight objects."""
        q = prefix + f"{experts_name}.{e}."
        if use_fp8:
            from ..models import quant
            from ..ops import fp8

            g = quant.load_fp8_weight(raw, q + "gate_proj.weight", 0, i0, i1)
            u = quant.load_fp8_weight(raw, q + "up_proj.weight", 0, i0, i1)
            return fp8.interleave_gate_up_fp8(g, u), quant.load_fp8_weight(raw, q + "down_proj.weight", 1, i0, i1)
        g = src.get(q + "gate_proj.weight", 0, i0, i1)
        u = src.get(q + "up_proj.weight", 0, i0, i1)
        return ref.interleave_gate_up(g, u), src.get(q + "down_proj.weight", 1, i0, i1)

    mats = [read_expert(e) for e in expert_ids]
    # `--enable_fused_shared_experts` (tensor-parallel experts): the shared expert joins the grouped GEMMs as
    # n_shared more experts that every token selects with weight 1, instead of two GEMMs of its own
    lw.fused_shared = 0
    ns = mc.n_shared
    if ns and model.extra.get("enable_fused_shared_experts") and not ep and not use_fp8 and not mc.shared_gate \
            and mc.shared_inter == ns * mc.inter:
        q = prefix + mc.shared_name + "."
        il = i1 - i0
        s0 = tp_range(mc.shared_inter, r, tp)[0]
        for j in range(ns):
            a, b = s0 + j * il, s0 + (j + 1) * il
            mats.append((ref.interleave_gate_up(src.get(q + "gate_proj.weight", 0, a, b),
                                                src.get(q + "up_proj.weight", 0, a, b)),
                         src.get(q + "down_proj.weight", 1, a, b)))
        lw.fused_shared = ns
    if use_fp8:
        # keep the experts in e4m3 with their block scales: grouped fp8 GEMMs, half the weight bytes
        from ..ops import fp8

        lw.w13 = fp8.Fp8Experts(fp8.stack_experts([m[0] for m in mats]), len(mats)).to(model.device)
        lw.w2 = fp8.Fp8Experts(fp8.stack_experts([m[1] for m in mats]), len(mats)).to(model.device)
    else:
        lw.w13 = dev(torch.stack([m[0] for m in mats]))
        lw.w2 = dev(torch.stack([m[1] for m in mats]))
    del mats
    lw.e0 = e0 if (ep and tp > 1) else 0
    lw.ep_world = tp if ep else 1
    lw.is_moe = True
    lw.ep_table = None
    if red_ids:
        from ..engine.redundancy import physical_table

        R = len(red_ids)
        lw.e0 = r * (e1 - e0 + R)                     # first PHYSICAL id of this rank
        lw.ep_table = physical_table(mc.num_experts, tp, r, red_ids).to(model.device)
        lw.ep_counter = torch.zeros(mc.num_experts, dtype=torch.int32, device=model.device)
        lw.ep_red_num, lw.ep_red_ids, lw.ep_layer = R, list(red_ids), layer_no
        lw.ep_read_expert = read_expert               # the manager re-reads experts from the checkpoint later
    if mc.n_shared and not lw.fused_shared:
        model._load_dense_ffn(lw, src, prefix + mc.shared_name + ".", mc.shared_inter)
        if mc.shared_gate:
            lw.shared_gate_w = dev(src.get(prefix + mc.shared_name + "_gate.weight"))
        lw.shared_gate_up_w, lw.shared_down_w, lw.shared_fused = lw.gate_up_w, lw.down_w, lw.gate_up_fused
        lw.gate_up_w = lw.down_w = None


def moe_ffn(model, lw, h, mc: MoEConfig, layer: int = -1, st=None):
    """Returns the per-rank partial sum [T, H] of routed (+ shared) experts, written where the TP reduction
    wants it."""
    T = h.shape[0]
    logits = ops.gemm(h, lw.router_w, epi="f32")
    if mc.scoring == "softmax" and mc.n_group <= 1:
        ids, w = moe_ops.topk_softmax(logits, mc.top_k, mc.renorm, mc.routed_scale)
    else:
        ids, w = moe_ops.grouped_topk(logits, lw.router_bias, mc.top_k, mc.n_group, mc.topk_group,
                                      mc.scoring == "sigmoid", mc.renorm, mc.routed_scale)
    rc = getattr(model, "route_capture", None)
    if rc is not None and st is not None and st.extra.get("balance") is None:   # --enable_return_routed_experts
        rc.capture(layer, ids, st.mem_index)
    out = model._partial_out(T)
    accumulate = False
    if lw.fused_shared:       # the shared expert's slices are experts E .. E + n - 1, chosen by every token
        extra = torch.arange(mc.num_experts, mc.num_experts + lw.fused_shared, dtype=ids.dtype, device=ids.device)
        ids = torch.cat([ids, extra.expand(T, -1)], dim=1)
        w = torch.cat([w, torch.ones((T, lw.fused_shared), dtype=w.dtype, device=w.device)], dim=1)
    elif mc.n_shared:
        if lw.shared_fused:
            act = ops.gemm(h, lw.shared_gate_up_w, epi="gated_" + mc.act)
        else:
            act = ops.gated_act(ops.gemm(h, lw.shared_gate_up_w), mc.act)
        ops.gemm(act, lw.shared_down_w, out=out)
        if mc.shared_gate:  # every rank scales its partial sum by the same (replicated) gate
            out.mul_(torch.sigmoid(torch.nn.functional.linear(h.float(), lw.shared_gate_w.float())).to(out.dtype))
        accumulate = True
    if getattr(lw, "ep_table", None) is not None:      # redundant experts: physical ids + hit counters
        ids = moe_ops.count_remap(ids, lw.ep_table, lw.ep_counter)
    epg = ep_group_of(model, mc)
    if epg is not None:
        fn = lambda hr, ir, wr, o: moe_ops.fused_experts(hr, lw.w13, lw.w2, ir, wr, mc.act, lw.e0, out=o)  # noqa: E731
        bound = int(getattr(model, "_ep_tokens_bound", 0) or 0)
        tp, t = model.ps.tp_size, model.ps.tp_rank
        if tp == 1:
            epg.moe(h, ids, w, fn, out=out, accumulate=accumulate, tokens_bound=bound)
            return out
        # tensor parallelism inside the replica: its ranks hold the same tokens, so each sends only its share of
        # them through the exchange and leaves the other rows of the partial sum to the other ranks; the replica's
        # reduction that follows adds the shares up
        per = -(-T // tp)
        lo, hi = min(t * per, T), min((t + 1) * per, T)
        if not accumulate:
            out.zero_()
        epg.moe(h[lo:hi], ids[lo:hi], w[lo:hi], fn, out=out[lo:hi], accumulate=True, tokens_bound=bound)
        return out
    moe_ops.fused_experts(h, lw.w13, lw.w2, ids, w, mc.act, lw.e0, out=out, accumulate=accumulate)
    return out


def ep_group_of(model, mc: MoEConfig):
    """The token exchange of a data-parallel + expert-parallel model (created on first use), else None."""
    if not (getattr(model, "ep", False) and model.ps.dp_size > 1 and model.ps.world_size > 1):
        return None
    g = getattr(model, "_ep_group", None)
    if g is None:
        from ..parallel.ep import EPGroup

        red = getattr(model, "redundancy_cfg", None)
        n_phys = mc.num_experts + model.ps.world_size * (red.num if red is not None else 0)
        g = model._ep_group = EPGroup(model.ps, model.hidden, mc.top_k, n_phys, model.batch_max_tokens)
    return g
