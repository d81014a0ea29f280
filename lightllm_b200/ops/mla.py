"""Multi-head latent attention (DeepSeek-V2/V3) over the latent KV pool.

The pool row of a token is `[c_kv (kv_lora_rank, already RMS-normalised) | k_pe (rope dim, rotated)]`,
one "head", shared by all query heads.  Attention runs in the absorbed form: the query is moved into
the latent space with W_UK (`q_lat = q_nope . W_UK`), scores are `q_lat . c_kv + q_pe . k_pe`, the
value read is the same `c_kv`, and W_UV brings the result back (`o = (P . c_kv) . W_UV^T`).

`mla_attention(...)` covers prefill (causal, cached-prefix aware) and decode; CUDA tensors use
`csrc/mla.cu`, CPU tensors the fp32 restatement below.

Reference: lightllm/models/deepseek2/layer_infer/transformer_layer_infer.py:75-214 and its MLA
Triton / FlashInfer back-ends.
"""
from __future__ import annotations

import math

import torch

from . import _count
from ._native import c_int, check, f32, i64, kernels, ptr, stream


def ref_mla_attention(q_lat, q_pe, kv_layer, req_to_token, b_req_idx, b_seq_len, cu_q, b_ready_len, kv_lora, scale):
    """q_lat [T, h, kv_lora], q_pe [T, h, rope]; kv_layer [slots, 1, kv_lora + rope].
    Request b owns query rows cu_q[b]:cu_q[b+1] at positions ready_len[b] + i; returns o_lat [T, h, kv_lora]."""
    T, h, _ = q_lat.shape
    out = torch.zeros(T, h, kv_lora, dtype=q_lat.dtype, device=q_lat.device)
    B = b_req_idx.shape[0]
    for b in range(B):
        s0, s1 = int(cu_q[b]), int(cu_q[b + 1])
        n = s1 - s0
        if n == 0:
            continue
        ready = int(b_ready_len[b])
        L = ready + n
        slots = req_to_token[int(b_req_idx[b]), :L].long()
        kv = kv_layer[slots, 0].float()
        c, kpe = kv[:, :kv_lora], kv[:, kv_lora:]
        s = torch.einsum("nhd,ld->hnl", q_lat[s0:s1].float(), c) + torch.einsum("nhr,lr->hnl", q_pe[s0:s1].float(), kpe)
        s = s * scale
        qpos = torch.arange(n, device=q_lat.device) + ready
        mask = torch.arange(L, device=q_lat.device)[None, :] <= qpos[:, None]
        s = s.masked_fill(~mask[None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[s0:s1] = torch.einsum("hnl,ld->nhd", p, c).to(q_lat.dtype)
    return out


def mla_attention(q_lat, q_pe, kv_layer, req_to_token, b_req_idx, b_seq_len, cu_q, b_ready_len, kv_lora, scale,
                  is_prefill: bool, max_q_len: int = 1, max_kv_len: int = 0, batch_of=None):
    if not q_lat.is_cuda:
        return ref_mla_attention(q_lat, q_pe, kv_layer, req_to_token, b_req_idx, b_seq_len, cu_q, b_ready_len, kv_lora,
                                 scale)
    T, h, _ = q_lat.shape
    rope = q_pe.shape[-1]
    assert kv_lora == 512 and rope == 64, "the MLA kernel is specialised for kv_lora_rank 512 / rope 64"
    assert q_lat.is_contiguous() and q_pe.stride(-1) == 1
    out = torch.empty((T, h, kv_lora), dtype=q_lat.dtype, device=q_lat.device)
    B = b_req_idx.shape[0]
    check(kernels().llb_mla_attention(ptr(q_lat), ptr(q_pe), i64(q_pe.stride(0)), i64(q_pe.stride(1)), ptr(kv_layer),
                                      ptr(req_to_token), i64(req_to_token.stride(0)), ptr(b_req_idx), ptr(cu_q),
                                      ptr(b_ready_len), ptr(batch_of), ptr(out), c_int(B), c_int(T), c_int(h),
                                      c_int(max_q_len),
                                      f32(scale), stream()), "mla_attention")
    _count()
    return out


def gemm_batched(a, w, out=None):
    """Per-head GEMM: a [T, h, K] (any row / head strides, unit inner stride), w [h, N, K] -> out [T, h, N].
    Used for the W_UK / W_UV absorption steps of MLA."""
    T, h, K = a.shape
    N = w.shape[1]
    if not a.is_cuda:
        return torch.einsum("thk,hnk->thn", a.float(), w.float()).to(a.dtype)
    from . import gemm_status

    assert a.stride(2) == 1 and w.is_contiguous()
    if out is None:
        out = torch.empty((T, h, N), dtype=a.dtype, device=a.device)
    check(kernels().llb_gemm_bf16_batched(ptr(a), i64(a.stride(0)), i64(a.stride(1)), ptr(w), ptr(out),
                                          i64(out.stride(0)), i64(out.stride(1)), c_int(T), c_int(N), c_int(K),
                                          c_int(h), ptr(gemm_status(a.device)), stream()), "gemm_batched")
    _count()
    return out
