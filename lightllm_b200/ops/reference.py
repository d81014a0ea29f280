"""Plain PyTorch fp32 restatements of every op: the numerics oracle for the CUDA kernels and
the execution path for CPU tensors (the CPU/gloo plumbing configuration runs on these).

Each function takes the same arguments as its CUDA counterpart in this package and works on
any device; math is done in fp32 and cast back to the input dtype at the end.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

GATE_UP_BLOCK = 32  # gate/up interleave granularity used by the fused gated GEMM epilogue


def rmsnorm(x, w, eps, w_offset=0.0):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + w_offset)
    return y.to(x.dtype)


def add_rmsnorm_(residual, x, w, eps, w_offset=0.0):
    residual.copy_((residual.float() + x.float()).to(residual.dtype))
    return rmsnorm(residual, w, eps, w_offset)


def _act(g, act):
    if act == "silu":
        return torch.nn.functional.silu(g)
    if act == "gelu":
        return torch.nn.functional.gelu(g, approximate="tanh")
    raise ValueError(act)


def gated_act(x, act="silu"):
    I = x.shape[-1] // 2
    xf = x.float()
    return (_act(xf[..., :I], act) * xf[..., I:]).to(x.dtype)


def interleave_gate_up(w_gate, w_up, block=GATE_UP_BLOCK):
    """[I, K] x2 -> [2I, K] with rows ordered [gate blk0 | up blk0 | gate blk1 | up blk1 ...]."""
    I, K = w_gate.shape[-2], w_gate.shape[-1]
    assert I % block == 0
    lead = w_gate.shape[:-2]
    g = w_gate.reshape(*lead, I // block, 1, block, K)
    u = w_up.reshape(*lead, I // block, 1, block, K)
    return torch.cat([g, u], dim=-3).reshape(*lead, 2 * I, K).contiguous()


def gated_act_interleaved(y, act="silu", block=GATE_UP_BLOCK):
    """y [T, 2I] produced with interleaved weights -> [T, I]."""
    T, N = y.shape
    v = y.float().view(T, N // (2 * block), 2, block)
    return (_act(v[:, :, 0, :], act) * v[:, :, 1, :]).reshape(T, N // 2).to(y.dtype)


def gemm(a, w, epi="store", residual=None, bias=None, out_dtype=None):
    """C = A . W^T with the epilogues of the tcgen05 GEMM. `w` is [N, K]."""
    acc = a.float() @ w.float().t()
    if bias is not None:
        acc = acc + bias.float()
    if epi == "store":
        return acc.to(out_dtype or a.dtype)
    if epi == "residual":
        return (acc + residual.float()).to(out_dtype or a.dtype)
    if epi == "f32":
        return acc
    if epi in ("gated_silu", "gated_gelu"):
        return gated_act_interleaved(acc, "silu" if epi == "gated_silu" else "gelu").to(out_dtype or a.dtype)
    raise ValueError(epi)


def embedding(ids, table, vocab_start, vocab_end):
    inside = (ids >= vocab_start) & (ids < vocab_end)
    local = torch.where(inside, ids - vocab_start, torch.zeros_like(ids))
    out = table[local]
    return out * inside.unsqueeze(-1).to(out.dtype)


def build_rope_cache(max_pos, rot_dim, theta=10000.0, scaling: Optional[dict] = None, device="cpu"):
    """cos/sin tables [max_pos, rot_dim/2] fp32, with the HF rope_scaling variants the reference
    supports (lightllm/models/llama/model.py:70-303): linear, dynamic NTK, llama3, yarn."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
    mscale = 1.0
    t = torch.arange(max_pos, dtype=torch.float64)
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type", "default"))
        factor = float(scaling.get("factor", 1.0))
        if kind == "linear":
            t = t / factor
        elif kind == "dynamic":
            orig = scaling.get("original_max_position_embeddings", max_pos)
            if max_pos > orig:
                base = theta * ((factor * max_pos / orig) - (factor - 1)) ** (rot_dim / (rot_dim - 2))
                inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
        elif kind == "llama3":
            lo = float(scaling.get("low_freq_factor", 1.0))
            hi = float(scaling.get("high_freq_factor", 4.0))
            orig = float(scaling.get("original_max_position_embeddings", 8192))
            wavelen = 2 * math.pi / inv_freq
            smooth = (orig / wavelen - lo) / (hi - lo)
            scaled = torch.where(
                wavelen > orig / lo,
                inv_freq / factor,
                torch.where(wavelen < orig / hi, inv_freq, (1 - smooth) * inv_freq / factor + smooth * inv_freq),
            )
            inv_freq = scaled
        elif kind == "yarn":
            orig = float(scaling.get("original_max_position_embeddings", 4096))
            beta_fast = float(scaling.get("beta_fast", 32))
            beta_slow = float(scaling.get("beta_slow", 1))

            def corr_dim(n_rot):
                return (rot_dim * math.log(orig / (n_rot * 2 * math.pi))) / (2 * math.log(theta))

            low = max(math.floor(corr_dim(beta_fast)), 0)
            high = min(math.ceil(corr_dim(beta_slow)), rot_dim - 1)
            if low == high:
                high += 0.001
            ramp = ((torch.arange(rot_dim // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
            mask = 1 - ramp
            inv_freq = inv_freq / factor * (1 - mask) + inv_freq * mask

            def get_mscale(scale, m=1.0):
                return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0

            m1 = scaling.get("mscale", 1.0)
            m2 = scaling.get("mscale_all_dim", 0.0)
            mscale = get_mscale(factor, m1) / get_mscale(factor, m2) if m2 else get_mscale(factor, m1)
            if "attention_factor" in scaling and scaling["attention_factor"] is not None:
                mscale = float(scaling["attention_factor"])
    freqs = torch.outer(t, inv_freq)
    cos = (freqs.cos() * mscale).float().to(device)
    sin = (freqs.sin() * mscale).float().to(device)
    return cos.contiguous(), sin.contiguous()


def rope_kv_scatter_(qkv, kv_layer, cos, sin, pos, slot, Hq, Hkv, D, rot_dim, q_norm_w=None, k_norm_w=None,
                     norm_eps=1e-6, norm_w_offset=0.0):
    """In-place RoPE of q inside `qkv` [T, (Hq+2Hkv)*D]; rotated K and V written to kv_layer[slot]."""
    T = qkv.shape[0]
    v3 = qkv.view(T, Hq + 2 * Hkv, D)
    q = v3[:, :Hq].float()
    k = v3[:, Hq:Hq + Hkv].float()
    v = v3[:, Hq + Hkv:]
    if q_norm_w is not None:
        q = rmsnorm(q.to(qkv.dtype), q_norm_w, norm_eps, norm_w_offset).float()
    if k_norm_w is not None:
        k = rmsnorm(k.to(qkv.dtype), k_norm_w, norm_eps, norm_w_offset).float()
    half = rot_dim // 2
    if rot_dim == 0:
        v3[:, :Hq] = q.to(qkv.dtype)
        kv_layer[slot.long(), :Hkv] = k.to(kv_layer.dtype)
        kv_layer[slot.long(), Hkv:] = v.to(kv_layer.dtype)
        return qkv
    c = cos[pos.long()].unsqueeze(1)
    s = sin[pos.long()].unsqueeze(1)

    def rot(x):
        x1, x2, rest = x[..., :half], x[..., half:rot_dim], x[..., rot_dim:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)

    v3[:, :Hq] = rot(q).to(qkv.dtype)
    kv_layer[slot.long(), :Hkv] = rot(k).to(kv_layer.dtype)
    kv_layer[slot.long(), Hkv:] = v.to(kv_layer.dtype)
    return qkv


def gqa_decode(q, kv_layer, req_to_token, b_req_idx, b_seq_len, Hq, Hkv, D, sm_scale=None):
    """q [B, Hq, D] -> out [B, Hq, D]; request b attends to its first b_seq_len[b] cached tokens."""
    B = q.shape[0]
    scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(D)
    G = Hq // Hkv
    out = torch.empty(B, Hq, D, dtype=q.dtype, device=q.device)
    for b in range(B):
        L = int(b_seq_len[b])
        slots = req_to_token[int(b_req_idx[b]), :L].long()
        k = kv_layer[slots, :Hkv].float()  # [L, Hkv, D]
        v = kv_layer[slots, Hkv:].float()
        qb = q[b].float().view(Hkv, G, D)
        s = torch.einsum("hgd,lhd->hgl", qb, k) * scale
        p = torch.softmax(s, dim=-1)
        out[b] = torch.einsum("hgl,lhd->hgd", p, v).reshape(Hq, D).to(q.dtype)
    return out


def gqa_prefill(q, kv_layer, req_to_token, b_req_idx, cu_q, b_ready_len, Hq, Hkv, D, sm_scale=None):
    """q [T, Hq, D] (new tokens of every request back to back); causal over cached prefix + new tokens."""
    scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(D)
    G = Hq // Hkv
    out = torch.empty_like(q)
    B = b_req_idx.shape[0]
    for b in range(B):
        s0, s1 = int(cu_q[b]), int(cu_q[b + 1])
        n = s1 - s0
        if n == 0:
            continue
        ready = int(b_ready_len[b])
        L = ready + n
        slots = req_to_token[int(b_req_idx[b]), :L].long()
        k = kv_layer[slots, :Hkv].float()
        v = kv_layer[slots, Hkv:].float()
        qb = q[s0:s1].float().view(n, Hkv, G, D)
        s = torch.einsum("nhgd,lhd->hgnl", qb, k) * scale
        qpos = torch.arange(n, device=q.device) + ready
        kpos = torch.arange(L, device=q.device)
        mask = kpos[None, :] <= qpos[:, None]
        s = s.masked_fill(~mask[None, None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("hgnl,lhd->nhgd", p, v).reshape(n, Hq, D)
        out[s0:s1] = o.to(q.dtype)
    return out


def apply_penalty_(logits, presence, frequency, repetition, cu, tok_ids, tok_cnt, mask_cu=None, mask_ids=None):
    B, V = logits.shape
    for b in range(B):
        if cu is not None:
            s, e = int(cu[b]), int(cu[b + 1])
            if e > s:
                ids = tok_ids[s:e].long()
                cnt = tok_cnt[s:e].float()
                x = logits[b, ids]
                rp = repetition[b]
                x = torch.where(x > 0, x / rp, x * rp)
                x = x - frequency[b] * cnt - presence[b]
                logits[b, ids] = x
        if mask_cu is not None:
            s, e = int(mask_cu[b]), int(mask_cu[b + 1])
            if e > s:
                logits[b, mask_ids[s:e].long()] = float("-inf")
    return logits


def sample(logits, temperature=None, top_p=None, top_k=None, seeds=None, steps=None):
    """Reference sampler: greedy rows exactly; random rows by filtered multinomial (the CUDA
    kernel draws from the same filtered distribution with a different generator)."""
    B, V = logits.shape
    ids = torch.empty(B, dtype=torch.int64, device=logits.device)
    lps = torch.empty(B, dtype=torch.float32, device=logits.device)
    for b in range(B):
        k = int(top_k[b]) if top_k is not None else 1
        t = float(temperature[b]) if temperature is not None else 1.0
        greedy = k == 1 or t < 1e-5
        x = logits[b].float() / (1.0 if greedy else t)
        logp = torch.log_softmax(x, dim=-1)
        if greedy:
            i = int(torch.argmax(x))
        else:
            keep = filtered_support(x, float(top_p[b]) if top_p is not None else 1.0, k)
            probs = torch.where(keep, logp.exp(), torch.zeros_like(logp))
            g = torch.Generator(device="cpu")
            g.manual_seed(int(seeds[b]) + int(steps[b]) * 1000003 if seeds is not None else b)
            i = int(torch.multinomial((probs / probs.sum()).cpu(), 1, generator=g))
        ids[b] = i
        lps[b] = logp[i]
    return ids, lps


def greedy_partials(logits, idx_off, splits):
    """[B, S, 3]: (max, arg-max global id as float bits, sum exp(x - max)) of S column slices."""
    B, V = logits.shape
    per = ((V + splits - 1) // splits + 3) & ~3
    out = torch.zeros((B, splits, 3), dtype=torch.float32, device=logits.device)
    for s in range(splits):
        i0, i1 = s * per, min(V, (s + 1) * per)
        if i1 <= i0:
            out[:, s, 0] = float("-inf")
            out[:, s, 1] = torch.tensor([0x7FFFFFFF], dtype=torch.int32).view(torch.float32)
            continue
        x = logits[:, i0:i1].float()
        m, i = x.max(dim=-1)
        out[:, s, 0] = m
        out[:, s, 1] = (i + i0 + idx_off).to(torch.int32).view(torch.float32)
        out[:, s, 2] = torch.exp(x - m[:, None]).sum(-1)
    return out


def greedy_merge(parts):
    R, B, S, _ = parts.shape
    p = parts.permute(1, 0, 2, 3).reshape(B, R * S, 3)
    m = p[..., 0]
    idx = p[..., 1].contiguous().view(torch.int32).to(torch.int64)
    best = m.max(dim=-1).values
    # ties go to the smallest token id, as in one pass over the whole row
    cand = torch.where(m == best[:, None], idx, torch.full_like(idx, 0x7FFFFFFF))
    ids = cand.min(dim=-1).values
    z = torch.where(p[..., 2] > 0, p[..., 2] * torch.exp(m - best[:, None]), torch.zeros_like(m)).sum(-1)
    return ids, -torch.log(z)


def filtered_support(x, top_p, top_k):
    """Boolean mask of the tokens that survive top-k then top-p on logits `x` (1-D)."""
    V = x.shape[0]
    probs = torch.softmax(x.float(), dim=-1)
    sp, si = torch.sort(probs, descending=True)
    keep_sorted = torch.ones(V, dtype=torch.bool, device=x.device)
    if 0 < top_k < V:
        keep_sorted &= torch.arange(V, device=x.device) < top_k
    if top_p < 1.0:
        csum = torch.cumsum(sp, dim=-1)
        keep_sorted &= (csum - sp) < top_p
    keep = torch.zeros(V, dtype=torch.bool, device=x.device)
    keep[si[keep_sorted]] = True
    return keep


def token_logprob(logits, ids):
    return torch.log_softmax(logits.float(), dim=-1).gather(1, ids.view(-1, 1).long()).squeeze(1)


def mla_rope_kv_scatter_(q3, kv_a, kv_layer, kv_norm_w, cos, sin, pos, slot, nope, rope, kv_lora, eps):
    """MLA counterpart of rope_kv_scatter_: rotates q3[:, :, nope:] in place (half-split layout), normalises
    the latent kv_a[:, :kv_lora], rotates k_pe = kv_a[:, kv_lora:], and writes [c_kv | k_pe] to kv_layer[slot, 0]."""
    half = rope // 2
    c = cos[pos.long()].unsqueeze(1)
    s = sin[pos.long()].unsqueeze(1)

    def rot(x):
        x1, x2 = x[..., :half], x[..., half:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)

    q3[:, :, nope:] = rot(q3[:, :, nope:].float()).to(q3.dtype)
    ckv = rmsnorm(kv_a[:, :kv_lora], kv_norm_w, eps)
    kpe = rot(kv_a[:, kv_lora:].float().unsqueeze(1)).squeeze(1).to(kv_a.dtype)
    kv_layer[slot.long(), 0, :kv_lora] = ckv.to(kv_layer.dtype)
    kv_layer[slot.long(), 0, kv_lora:] = kpe.to(kv_layer.dtype)
    return q3


def layernorm(x, w, b, eps, residual=None):
    """LayerNorm over the last dim; with `residual` the sum x + residual is normalised and stored back."""
    if residual is not None:
        residual.copy_((residual.float() + x.float()).to(residual.dtype))
        x = residual
    y = torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), w.float(), None if b is None else b.float(), eps)
    return y.to(x.dtype)


ACT_KINDS = {"silu": 0, "gelu_tanh": 1, "gelu_pytorch_tanh": 1, "gelu_new": 1, "gelu_fast": 1, "gelu": 2, "relu": 3,
             "scale": 4}


def act_(x, kind: str, alpha: float = 1.0):
    f = x.float()
    k = ACT_KINDS[kind]
    if k == 0:
        f = torch.nn.functional.silu(f)
    elif k == 1:
        f = torch.nn.functional.gelu(f, approximate="tanh")
    elif k == 2:
        f = torch.nn.functional.gelu(f)
    elif k == 3:
        f = torch.relu(f)
    else:
        f = f * alpha
    x.copy_(f.to(x.dtype))
    return x


def attention_generic(q, kv_layer, req_to_token, b_req_idx, pos, batch_of, Hq, Hkv, D, sm_scale, window=0,
                      softcap=0.0, alibi=None, sinks=None):
    """q [T, Hq, D]; token t belongs to request row batch_of[t] (t itself when None) at position pos[t] and
    attends keys max(0, pos - window + 1) .. pos of that request."""
    T = q.shape[0]
    out = torch.zeros(T, Hq, D, dtype=q.dtype, device=q.device)
    G = Hq // Hkv
    for t in range(T):
        b = int(batch_of[t]) if batch_of is not None else t
        p = int(pos[t])
        j0 = max(0, p - window + 1) if window > 0 else 0
        slots = req_to_token[int(b_req_idx[b]), j0:p + 1].long()
        k = kv_layer[slots, :Hkv].float().repeat_interleave(G, dim=1)      # [L, Hq, D]
        v = kv_layer[slots, Hkv:2 * Hkv].float().repeat_interleave(G, dim=1)
        s = torch.einsum("hd,lhd->hl", q[t].float(), k) * sm_scale
        if softcap > 0:
            s = softcap * torch.tanh(s / softcap)
        if alibi is not None:
            rel = torch.arange(j0, p + 1, device=q.device, dtype=torch.float32) - p
            s = s + alibi.float()[:, None] * rel[None, :]
        if sinks is not None:
            s = torch.cat([s, sinks.float()[:, None]], dim=1)
            pr = torch.softmax(s, dim=-1)[:, :-1]
        else:
            pr = torch.softmax(s, dim=-1)
        out[t] = torch.einsum("hl,lhd->hd", pr, v).to(q.dtype)
    return out
