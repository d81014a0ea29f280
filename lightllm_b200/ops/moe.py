"""MoE operators: routing (softmax top-k, DeepSeek grouped top-k), expert-sorted layout, grouped
tcgen05 GEMMs, weighted combine.  CUDA tensors run the kernels of `csrc/moe.cu` / `gemm_tcgen05.cu`;
CPU tensors run the fp32 PyTorch restatements below (also the test oracle).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _count, gemm_status
from . import reference as ref
from ._native import c_int, check, f32, i64, kernels, ptr, stream


# ---------------------------------------------------------------- references
def ref_topk_softmax(logits, k, renorm=True, scale=1.0):
    p = torch.softmax(logits.float(), dim=-1)
    w, ids = torch.topk(p, k, dim=-1)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return ids.to(torch.int32), (w * scale).float()


def ref_grouped_topk(logits, bias, k, n_group, topk_group, use_sigmoid=True, renorm=True, scale=1.0):
    x = logits.float()
    scores = torch.sigmoid(x) if use_sigmoid else torch.softmax(x, dim=-1)
    T, E = scores.shape
    biased = scores + (bias.float() if bias is not None else 0.0)
    g = biased.view(T, n_group, E // n_group)
    gscore = g.topk(2, dim=-1)[0].sum(-1) if bias is not None else g.max(-1)[0]
    gidx = gscore.topk(topk_group, dim=-1)[1]
    gmask = torch.zeros_like(gscore).scatter_(1, gidx, 1.0)
    mask = gmask.unsqueeze(-1).expand(T, n_group, E // n_group).reshape(T, E)
    masked = biased.masked_fill(mask == 0, float("-inf"))
    ids = masked.topk(k, dim=-1)[1]
    w = scores.gather(1, ids)
    if renorm:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return ids.to(torch.int32), (w * scale).float()


def _swiglu_oai(h, alpha=1.702, limit=7.0):
    """h [.., 2I] with gate / up interleaved in 32-column blocks (GPT-OSS clamped SwiGLU)."""
    n = h.shape[-1] // 64
    hv = h.reshape(*h.shape[:-1], n, 2, 32)
    g, u = hv[..., 0, :].clamp(max=limit), hv[..., 1, :].clamp(min=-limit, max=limit)
    return ((u + 1) * g * torch.sigmoid(alpha * g)).reshape(*h.shape[:-1], n * 32)


def ref_fused_experts(x, w13, w2, ids, weights, act="silu", e0=0, interleaved=True, b13=None, b2=None):
    """x [T,H]; w13 [E_local, 2I, H] (gate/up interleaved in 32-row blocks when `interleaved`), w2 [E_local, H, I];
    experts outside [e0, e0+E_local) contribute nothing (expert parallel shard)."""
    T, H = x.shape
    E_local = w13.shape[0]
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    xf = x.float()
    for e in range(E_local):
        sel = (ids == e + e0)
        if not sel.any():
            continue
        tok, slot = sel.nonzero(as_tuple=True)
        h = xf[tok] @ w13[e].float().t()
        if b13 is not None:
            h = h.to(x.dtype).float() + b13[e].float()
        if act == "swiglu_oai":
            a = _swiglu_oai(h)
        elif interleaved:
            a = ref.gated_act_interleaved(h, act).float()
        else:
            a = ref.gated_act(h, act).float()
        a = a.to(x.dtype).float()
        y = (a @ w2[e].float().t()).to(x.dtype).float()
        if b2 is not None:
            y = (y + b2[e].float()).to(x.dtype).float()
        out.index_add_(0, tok, y * weights[tok, slot].unsqueeze(-1))
    return out.to(x.dtype)


# ---------------------------------------------------------------- kernels
def topk_softmax(logits, k, renorm=True, scale=1.0):
    if not logits.is_cuda:
        return ref_topk_softmax(logits, k, renorm, scale)
    T, E = logits.shape
    ids = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    dt = {torch.float32: 0, torch.bfloat16: 1}[logits.dtype]
    check(kernels().llb_topk_softmax(ptr(logits), c_int(dt), i64(logits.stride(0)), c_int(T), c_int(E), c_int(k),
                                     c_int(1 if renorm else 0), f32(scale), ptr(ids), ptr(w), stream()), "topk_softmax")
    _count()
    return ids, w


def grouped_topk(logits, bias, k, n_group, topk_group, use_sigmoid=True, renorm=True, scale=1.0):
    if not logits.is_cuda:
        return ref_grouped_topk(logits, bias, k, n_group, topk_group, use_sigmoid, renorm, scale)
    T, E = logits.shape
    ids = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    dt = {torch.float32: 0, torch.bfloat16: 1}[logits.dtype]
    if bias is not None:
        assert bias.dtype == torch.float32
    check(kernels().llb_grouped_topk(ptr(logits), c_int(dt), i64(logits.stride(0)), ptr(bias), c_int(T), c_int(E),
                                     c_int(k), c_int(n_group), c_int(topk_group), c_int(1 if use_sigmoid else 0),
                                     c_int(1 if renorm else 0), f32(scale), ptr(ids), ptr(w), stream()), "grouped_topk")
    _count()
    return ids, w


def max_padded_rows(T: int, k: int, E_local: int) -> int:
    """Upper bound of the expert-sorted row count (every expert's rows padded to 128)."""
    n = T * k
    worst = n + min(E_local, n) * 127
    return ((worst + 127) // 128) * 128


class MoeLayout:
    """Device-side description of the expert-sorted layout of one step (no host sync)."""

    __slots__ = ("sorted_pair", "pair_row", "mblock_expert", "expert_off", "total_rows", "m_pad", "k")


def moe_align(ids, E_local: int, e0: int = 0) -> MoeLayout:
    T, k = ids.shape
    m_pad = max_padded_rows(T, k, E_local)
    dev = ids.device
    lay = MoeLayout()
    lay.m_pad, lay.k = m_pad, k
    lay.sorted_pair = torch.empty(m_pad, dtype=torch.int32, device=dev)
    lay.pair_row = torch.empty(T * k, dtype=torch.int32, device=dev)
    lay.mblock_expert = torch.empty(m_pad // 128, dtype=torch.int32, device=dev)
    lay.expert_off = torch.empty(E_local + 1, dtype=torch.int32, device=dev)
    lay.total_rows = torch.empty(1, dtype=torch.int32, device=dev)
    check(kernels().llb_moe_align(ptr(ids), c_int(T * k), c_int(e0), c_int(E_local), c_int(m_pad), ptr(lay.sorted_pair),
                                  ptr(lay.pair_row), ptr(lay.mblock_expert), ptr(lay.expert_off), ptr(lay.total_rows),
                                  stream()), "moe_align")
    _count()
    return lay


def count_remap(ids, table, counter=None):
    """ids [T, k] int32 (router's expert ids) -> table[ids] (ids outside the table become -1); counter[e] += number of
    times e was chosen.  One launch; CPU: torch ops."""
    if not ids.is_cuda:
        flat = ids.reshape(-1).long()
        ok = (flat >= 0) & (flat < table.numel())
        if counter is not None:
            counter += torch.bincount(flat[ok], minlength=counter.numel()).to(counter.dtype)
        out = torch.full_like(flat, -1, dtype=torch.int32)
        out[ok] = table[flat[ok]]
        return out.view_as(ids)
    assert ids.dtype == torch.int32 and table.dtype == torch.int32 and ids.is_contiguous()
    out = torch.empty_like(ids)
    check(kernels().llb_moe_count_remap(ptr(ids), c_int(ids.numel()), ptr(table), c_int(table.numel()),
                                        ptr(counter) if counter is not None else None, ptr(out), stream()),
          "moe_count_remap")
    _count()
    return out


def gemm_grouped(a_sorted, w_stacked, mblock_expert, n_per_expert: int, epi: str = "store", out=None, bn: int = 0):
    """a_sorted [M_pad, K] bf16, w_stacked [E, N, K] bf16 -> [M_pad, N] (or [M_pad, N/2] gated)."""
    from . import EPI_CODES

    M_pad, K = a_sorted.shape
    E, N = w_stacked.shape[0], w_stacked.shape[1]
    assert N == n_per_expert and w_stacked.is_contiguous()
    n_out = N // 2 if epi.startswith("gated") else N
    if out is None:
        out = torch.empty((M_pad, n_out), dtype=a_sorted.dtype, device=a_sorted.device)
    check(kernels().llb_gemm_bf16_grouped(ptr(a_sorted), i64(a_sorted.stride(0)), ptr(w_stacked), i64(K), ptr(out),
                                          i64(out.stride(0)), ptr(mblock_expert), c_int(M_pad), c_int(N), c_int(K),
                                          c_int(E), c_int(EPI_CODES[epi]), c_int(bn), ptr(gemm_status(a_sorted.device)),
                                          stream()), "gemm_grouped")
    _count()
    return out


def fused_experts(x, w13, w2, ids, weights, act="silu", e0: int = 0, out=None, accumulate: bool = False,
                  b13=None, b2=None):
    """Routed expert FFN:  out[t] (+)= sum_k w[t,k] * down_e( act(gate_e(x_t)) * up_e(x_t) ),  e = ids[t,k].

    w13 [E_local, 2I, H] with gate/up rows interleaved in 32-row blocks, w2 [E_local, H, I].  On CUDA: align
    -> gather -> grouped GEMM with gated epilogue -> grouped GEMM -> weighted combine (5 launches)."""
    fp8_w = type(w13).__name__ == "Fp8Experts"
    if not x.is_cuda:
        if fp8_w:  # CPU: same arithmetic with the de-quantised weights
            w13, w2 = w13.dequant().to(x.dtype), w2.dequant().to(x.dtype)
        r = ref_fused_experts(x, w13, w2, ids, weights, act, e0, b13=b13, b2=b2)
        if out is not None:
            if accumulate:
                out.add_(r)
            else:
                out.copy_(r)
            return out
        return r
    T, H = x.shape
    E_local, N13, _ = w13.shape
    I = N13 // 2
    k = ids.shape[1]
    lay = moe_align(ids, E_local, e0)
    a = torch.empty((lay.m_pad, H), dtype=x.dtype, device=x.device)
    check(kernels().llb_moe_gather(ptr(a), ptr(x), ptr(lay.sorted_pair), ptr(lay.total_rows), c_int(k), c_int(H),
                                   i64(x.stride(0)), c_int(lay.m_pad), stream()), "moe_gather")
    _count()
    if fp8_w:
        # block-scaled e4m3 experts: quantise the gathered rows per token group, grouped fp8 GEMM with the SwiGLU
        # epilogue, quantise again, grouped fp8 GEMM (reference: lightllm/common/basemodel/layer_weights/
        # meta_weights/fused_moe/impl/deepgemm_impl.py, the masked / contiguous m_grouped_fp8_gemm_nt path)
        from . import fp8

        assert act == "silu" and b13 is None and b2 is None, "fp8 experts: SwiGLU without bias"
        aq, asc = fp8.quant_act(a)
        h = fp8.gemm_fp8_quantized(aq, asc, w13.w, "gated_silu", mblock_expert=lay.mblock_expert, n_per_expert=N13)
        hq, hsc = fp8.quant_act(h)
        y = fp8.gemm_fp8_quantized(hq, hsc, w2.w, "store", mblock_expert=lay.mblock_expert, n_per_expert=H)
    elif b13 is None and act in ("silu", "gelu"):
        h = gemm_grouped(a, w13, lay.mblock_expert, N13, epi="gated_" + act)
    else:  # biased experts / clamped SwiGLU: plain grouped GEMM, then bias + activation in one pass
        h13 = gemm_grouped(a, w13, lay.mblock_expert, N13, epi="store")
        h = torch.empty((lay.m_pad, I), dtype=x.dtype, device=x.device)
        kind = {"silu": 0, "gelu": 1, "swiglu_oai": 2}[act]
        check(kernels().llb_moe_bias_act(ptr(h13), ptr(b13), ptr(lay.mblock_expert), ptr(h), c_int(lay.m_pad), c_int(I),
                                         c_int(kind), f32(1.702), f32(7.0), stream()), "moe_bias_act")
        _count()
    if not fp8_w:
        y = gemm_grouped(h, w2, lay.mblock_expert, H, epi="store")
    if b2 is not None:
        check(kernels().llb_moe_add_bias(ptr(y), ptr(b2), ptr(lay.mblock_expert), c_int(lay.m_pad), c_int(H), stream()),
              "moe_add_bias")
        _count()
    if out is None:
        out = torch.empty((T, H), dtype=x.dtype, device=x.device)
        accumulate = False
    check(kernels().llb_moe_combine(ptr(out), ptr(y), ptr(lay.pair_row), ptr(weights), c_int(T), c_int(k), c_int(H),
                                    c_int(1 if accumulate else 0), stream()), "moe_combine")
    _count()
    return out
