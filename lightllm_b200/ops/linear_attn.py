"""Gated DeltaNet linear attention (Qwen3-Next / Qwen3.5 hybrid layers) on torch ops.

Per head the layer keeps a matrix state S [dk, dv] and updates it token by token:

    S <- exp(g_t) * S                               (decay)
    d  = beta_t * (v_t - S^T k_t)                   (what the state does not predict yet)
    S <- S + k_t d^T ,   o_t = S^T q_t

with q, k l2-normalised and q scaled by dk^-1/2.  `gated_delta_step` is that recurrence for one token of every
request of a decode batch; `gated_delta_chunked` processes a whole prompt in chunks of 64 tokens with matrix
products: inside a chunk with start state S0 and cumulative log-decay G_i the corrections D solve the unit lower
triangular system (I + A) D = beta * (V - exp(G) * K S0), A_ij = beta_i exp(G_i - G_j) (k_i . k_j) for j < i; then
O = exp(G) * Q S0 + (M * Q K^T) D with M_ij = exp(G_i - G_j) for j <= i, and the chunk's end state is
exp(G_C) S0 + (exp(G_C - G) * K)^T D.  A depthwise causal convolution (kernel 4, SiLU) runs over q, k, v first; its
state is the last kernel-1 inputs.

Reference: lightllm/models/qwen3next/ (triton_kernel/fla/*, causal_conv1d) and the flash-linear-attention kernels
it wraps.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def causal_conv_prefill(x: torch.Tensor, state: torch.Tensor, w: torch.Tensor):
    """x [T, C] new inputs of one request, state [C, K-1] (previous inputs, zeros for a fresh request), w [C, K].
    Returns (silu(conv) [T, C], new state [C, K-1])."""
    K = w.shape[1]
    full = torch.cat([state.to(x.dtype), x.t()], dim=1)           # [C, K-1+T]
    y = F.conv1d(full.unsqueeze(0), w.to(x.dtype).unsqueeze(1), groups=w.shape[0])[0]   # [C, T]
    return F.silu(y).t(), full[:, -(K - 1):].contiguous()


def causal_conv_step(x: torch.Tensor, state: torch.Tensor, w: torch.Tensor):
    """One token per request: x [B, C], state [B, C, K-1] -> (silu(conv) [B, C], new state)."""
    full = torch.cat([state.to(x.dtype), x.unsqueeze(-1)], dim=-1)  # [B, C, K]
    y = (full * w.to(x.dtype).unsqueeze(0)).sum(-1)
    return F.silu(y), full[:, :, 1:].contiguous()


def gated_delta_naive(q, k, v, g, beta, S0=None):
    """Token-by-token recurrence (the definition): q, k [T, H, dk], v [T, H, dv], g, beta [T, H] -> (o [T, H, dv], S)."""
    T, H, dk = k.shape
    dv = v.shape[-1]
    q = l2norm(q.float()) * dk ** -0.5
    k = l2norm(k.float())
    v, g, beta = v.float(), g.float(), beta.float()
    S = torch.zeros(H, dk, dv, dtype=torch.float32, device=q.device) if S0 is None else S0.float().clone()
    o = torch.empty(T, H, dv, dtype=torch.float32, device=q.device)
    for t in range(T):
        S = S * g[t].exp().view(H, 1, 1)
        d = (v[t] - torch.einsum("hkv,hk->hv", S, k[t])) * beta[t].unsqueeze(-1)
        S = S + k[t].unsqueeze(-1) * d.unsqueeze(-2)
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def gated_delta_step(q, k, v, g, beta, S):
    """One token of each request: q, k [B, H, dk], v [B, H, dv], g, beta [B, H], S [B, H, dk, dv] fp32.
    Returns (o [B, H, dv] fp32, new S)."""
    dk = k.shape[-1]
    q = l2norm(q.float()) * dk ** -0.5
    k = l2norm(k.float())
    S = S * g.float().exp().unsqueeze(-1).unsqueeze(-1)
    d = (v.float() - torch.einsum("bhkv,bhk->bhv", S, k)) * beta.float().unsqueeze(-1)
    S = S + k.unsqueeze(-1) * d.unsqueeze(-2)
    return torch.einsum("bhkv,bhk->bhv", S, q), S


def gated_delta_chunked(q, k, v, g, beta, S0=None, chunk: int = 64):
    """A prompt (or a chunk of it) of one request: shapes as `gated_delta_naive`; S0 [H, dk, dv] fp32 or None."""
    T, H, dk = k.shape
    dv = v.shape[-1]
    dev = q.device
    q = (l2norm(q.float()) * dk ** -0.5).transpose(0, 1)   # [H, T, dk]
    k = l2norm(k.float()).transpose(0, 1)
    v = v.float().transpose(0, 1)
    g = g.float().t()                                       # [H, T]
    beta = beta.float().t()
    S = torch.zeros(H, dk, dv, dtype=torch.float32, device=dev) if S0 is None else S0.float().clone()
    out = torch.empty(H, T, dv, dtype=torch.float32, device=dev)
    for s in range(0, T, chunk):
        e = min(s + chunk, T)
        C = e - s
        qc, kc, vc, bc = q[:, s:e], k[:, s:e], v[:, s:e], beta[:, s:e]
        G = g[:, s:e].cumsum(-1)                                     # [H, C], <= 0 and decreasing
        ratio = (G.unsqueeze(-1) - G.unsqueeze(-2))                  # G_i - G_j
        lower = torch.tril(torch.ones(C, C, dtype=torch.bool, device=dev))
        M = torch.where(lower, ratio, torch.full_like(ratio, float("-inf"))).exp()   # exp(G_i - G_j), j <= i
        kk = kc @ kc.transpose(-1, -2)                               # k_i . k_j
        A = (bc.unsqueeze(-1) * M * kk).tril(-1)
        eG = G.exp().unsqueeze(-1)
        rhs = bc.unsqueeze(-1) * (vc - eG * (kc @ S))
        eye = torch.eye(C, dtype=torch.float32, device=dev).expand(H, C, C)
        D = torch.linalg.solve_triangular(eye + A, rhs, upper=False, unitriangular=True)
        out[:, s:e] = eG * (qc @ S) + (M * (qc @ kc.transpose(-1, -2))) @ D
        tail = (G[:, -1:] - G).exp().unsqueeze(-1)                   # exp(G_C - G_j)
        S = G[:, -1].exp().view(H, 1, 1) * S + (kc * tail).transpose(-1, -2) @ D
    return out.transpose(0, 1), S


def conv_and_delta_step(mixed, conv_state, conv_w_f32, ssm_state, req, g, beta, nk: int, nv: int, dk: int, dv: int):
    """The decode step of one Gated DeltaNet layer for a batch, two kernels (csrc/linear_attn.cu): convolution step
    over the q / k / v channels, then per (request, value head) the normalisation of q and k, the state update and the
    read-out, with the state row strips held in registers (one read and one write of the state).  Updates
    `conv_state [slots, C, K-1]` and `ssm_state [slots, nv, dk, dv]` (fp32 or bf16) in place at rows `req`.

    mixed [B, C] fp32, conv_w_f32 [C, K] fp32, req [B] int32, g / beta [B, nv] fp32 -> core [B, nv, dv] fp32."""
    import ctypes

    from . import _count
    from ._native import check, kernels, ptr, stream

    B, C = mixed.shape
    K = conv_w_f32.shape[1]
    assert mixed.dtype == torch.float32 and mixed.is_contiguous() and C == 2 * nk * dk + nv * dv
    assert conv_state.is_contiguous() and ssm_state.is_contiguous() and req.dtype == torch.int32
    assert conv_state.dtype in (torch.float32, torch.bfloat16) and ssm_state.dtype in (torch.float32, torch.bfloat16)
    g, beta = g.contiguous(), beta.contiguous()
    y = torch.empty_like(mixed)
    ci = ctypes.c_int
    check(kernels().llb_gdn_conv_step(ptr(mixed), ptr(conv_state), ci(int(conv_state.dtype == torch.bfloat16)),
                                      ptr(conv_w_f32), ptr(req), ptr(y), ci(B), ci(C), ci(K), stream()),
          "gdn_conv_step")
    core = torch.empty((B, nv, dv), dtype=torch.float32, device=mixed.device)
    check(kernels().llb_gdn_recurrent_step(ptr(y), ptr(g), ptr(beta), ptr(ssm_state),
                                           ci(int(ssm_state.dtype == torch.bfloat16)), ptr(req), ptr(core), ci(B),
                                           ci(nk), ci(nv), ci(dk), ci(dv), stream()), "gdn_recurrent_step")
    _count(2)
    return core


def step_kernel_supported(dk: int, dv: int, K: int) -> bool:
    """Shapes the decode-step kernels take: the value head fits a CTA in whole warps (dv a multiple of 32, at most
    256) and a thread's strip of a state column fits its registers (dk <= 64 x (256 // dv))."""
    return dv % 32 == 0 and 32 <= dv <= 256 and 1 <= K <= 16 and 1 <= dk <= 64 * (256 // dv)


def rmsnorm_gated(x: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """norm(x) * w * silu(z) over the last dimension (the norm sees x alone; z only gates)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (w.float() * y * F.silu(z.float())).to(z.dtype)
