"""Operator layer: every hot op as a hand-written sm_100a kernel (CUDA tensors) with a plain
PyTorch fp32 restatement (`ops.reference`) that serves CPU tensors and the numerics tests.

CUDA tensors always take the kernel path; if the native library is missing the call raises.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from . import kv_quant
from . import reference as ref
from ._native import NativeError, c_int, c_void_p, check, f32, i64, kernels, ptr, stream

EPI_CODES = {"store": 0, "residual": 1, "gated_silu": 2, "f32": 3, "gated_gelu": 4}

import os as _os

_GEMM_DEBUG_TORCH = _os.environ.get("LLB_GEMM_DEBUG_TORCH", "0") == "1"

# launch counter: the number of kernels of this package launched (claimed in bench output)
_launches = 0


def launch_count() -> int:
    return _launches


def _count(n=1):
    global _launches
    _launches += n


def _is_cuda(t) -> bool:
    return t.is_cuda


def _req_bf16(*ts):
    for t in ts:
        if t is not None and t.dtype != torch.bfloat16:
            raise NativeError(f"CUDA kernels take bf16 tensors, got {t.dtype}")


# --------------------------------------------------------------------------------------
def rmsnorm(x, w, eps: float, w_offset: float = 0.0, out=None):
    if not _is_cuda(x):
        return ref.rmsnorm(x, w, eps, w_offset)
    _req_bf16(x, w)
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    T = x2.shape[0]
    if out is None:
        out = torch.empty((T, H), dtype=x.dtype, device=x.device)
    check(kernels().llb_rmsnorm(ptr(out), ptr(x2), ptr(w), c_int(T), c_int(H), f32(eps), f32(w_offset),
                                i64(x2.stride(0)), i64(out.stride(0)), stream()), "rmsnorm")
    _count()
    return out.view(*x.shape[:-1], H)


def add_rmsnorm_(residual, x, w, eps: float, w_offset: float = 0.0, out=None):
    """residual += x (in place); returns rmsnorm(residual)."""
    if not _is_cuda(x):
        return ref.add_rmsnorm_(residual, x, w, eps, w_offset)
    _req_bf16(residual, x, w)
    assert residual.is_contiguous() and x.is_contiguous()
    T, H = x.shape
    if out is None:
        out = torch.empty_like(x)
    check(kernels().llb_add_rmsnorm(ptr(out), ptr(residual), ptr(x), ptr(w), c_int(T), c_int(H), f32(eps),
                                    f32(w_offset), stream()), "add_rmsnorm")
    _count()
    return out


def gated_act(x, act: str = "silu", out=None):
    if not _is_cuda(x):
        return ref.gated_act(x, act)
    _req_bf16(x)
    assert x.is_contiguous()
    T, N = x.shape
    if out is None:
        out = torch.empty((T, N // 2), dtype=x.dtype, device=x.device)
    check(kernels().llb_gated_act(ptr(out), ptr(x), c_int(T), c_int(N // 2), c_int(0 if act == "silu" else 1),
                                  stream()), "gated_act")
    _count()
    return out


def rope_kv_scatter_(qkv, kv_layer, cos, sin, pos, slot, Hq, Hkv, D, rot_dim=None, q_norm_w=None, k_norm_w=None,
                     norm_eps=1e-6, norm_w_offset=0.0):
    """rot_dim None = full head; 0 = no rotation (ALiBi / learned positions: K and V are only scattered)."""
    rot_dim = D if rot_dim is None else rot_dim
    if isinstance(kv_layer, kv_quant.QuantKVLayer):
        return kv_quant.rope_kv_scatter_(qkv, kv_layer, cos, sin, pos, slot, Hq, Hkv, D, rot_dim, q_norm_w, k_norm_w,
                                         norm_eps, norm_w_offset)
    if not _is_cuda(qkv):
        return ref.rope_kv_scatter_(qkv, kv_layer, cos, sin, pos, slot, Hq, Hkv, D, rot_dim, q_norm_w, k_norm_w,
                                    norm_eps, norm_w_offset)
    _req_bf16(qkv, kv_layer, q_norm_w, k_norm_w)
    assert qkv.stride(-1) == 1 and kv_layer.is_contiguous()
    assert pos.dtype == torch.int32 and slot.dtype == torch.int32
    T = qkv.shape[0]
    if D not in (64, 128, 256) or rot_dim % 16 != 0:
        assert q_norm_w is None and k_norm_w is None, "q/k norm needs a head size of 64, 128 or 256"
        assert rot_dim == 0 or (cos.dtype == torch.float32 and cos.shape[-1] == rot_dim // 2)
        check(kernels().llb_rope_kv_scatter_generic(ptr(qkv), ptr(kv_layer), ptr(cos), ptr(sin), ptr(pos), ptr(slot),
                                                    c_int(T), c_int(Hq), c_int(Hkv), c_int(D), c_int(rot_dim),
                                                    i64(qkv.stride(0)), stream()), "rope_kv_scatter_generic")
        _count()
        return qkv
    assert rot_dim == 0 or (cos.dtype == torch.float32 and cos.shape[-1] == rot_dim // 2)
    check(kernels().llb_rope_kv_scatter(ptr(qkv), ptr(kv_layer), ptr(cos), ptr(sin), ptr(pos), ptr(slot),
                                        ptr(q_norm_w), ptr(k_norm_w), f32(norm_eps), f32(norm_w_offset), c_int(T),
                                        c_int(Hq), c_int(Hkv), c_int(D), c_int(rot_dim), i64(qkv.stride(0)),
                                        stream()), "rope_kv_scatter")
    _count()
    return qkv


def mla_rope_kv_scatter_(q3, kv_a, kv_layer, kv_norm_w, cos, sin, pos, slot, nope, rope, kv_lora, eps):
    """RoPE on the rope part of q (in place), RMSNorm of the kv latent, RoPE of k_pe, scatter of
    [c_kv | k_pe] into the latent pool -- one launch."""
    if not _is_cuda(q3):
        return ref.mla_rope_kv_scatter_(q3, kv_a, kv_layer, kv_norm_w, cos, sin, pos, slot, nope, rope, kv_lora, eps)
    _req_bf16(q3, kv_a, kv_layer, kv_norm_w)
    T, hq, qd = q3.shape
    assert q3.stride(2) == 1 and kv_a.stride(1) == 1 and kv_layer.is_contiguous()
    check(kernels().llb_mla_rope_kv_scatter(ptr(q3), i64(q3.stride(0)), i64(q3.stride(1)), ptr(kv_a),
                                            i64(kv_a.stride(0)), ptr(kv_layer), ptr(kv_norm_w), ptr(cos), ptr(sin),
                                            ptr(pos), ptr(slot), c_int(T), c_int(hq), c_int(nope), c_int(rope),
                                            c_int(kv_lora), f32(eps), stream()), "mla_rope_kv_scatter")
    _count()
    return q3


def embedding(ids, table, vocab_start: int = 0, vocab_end: Optional[int] = None):
    vocab_end = vocab_start + table.shape[0] if vocab_end is None else vocab_end
    if not _is_cuda(table):
        return ref.embedding(ids, table, vocab_start, vocab_end)
    _req_bf16(table)
    assert ids.dtype == torch.int64 and ids.is_contiguous()
    T, H = ids.shape[0], table.shape[1]
    out = torch.empty((T, H), dtype=table.dtype, device=table.device)
    check(kernels().llb_embedding(ptr(out), ptr(ids), ptr(table), c_int(T), c_int(H), c_int(vocab_start),
                                  c_int(vocab_end), stream()), "embedding")
    _count()
    return out


# --------------------------------------------------------------------------------------
_status_words = {}


def gemm_status(device) -> torch.Tensor:
    """Device int that receives a code if a bounded wait inside a GEMM ran out (0 = healthy)."""
    key = torch.device(device).index or 0
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[key]


_sk_scratch = {}


def _stream_k_scratch(device):
    """fp32 partial-tile buffer and per-tile arrival counters for the stream-K schedule (per device;
    all GEMMs of a stream share them, which is safe because they run back to back on that stream)."""
    key = torch.device(device).index or 0
    cur = _sk_scratch.get(key)
    if cur is None:
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        # counters: [0, 8192) stream-K tiles (self-resetting); [8192, 16384) arrival counters of the split-K kernel
        cur = (torch.empty(sms * 2 * 128 * 256, dtype=torch.float32, device=device),
               torch.zeros(16384, dtype=torch.int32, device=device))
        _sk_scratch[key] = cur
    return cur


class TiledWeight:
    """A [N, K] weight stored as [N/128][K/64][128][64]: every 128-row x 64-column tile (what one TMA box of
    the GEMM kernels fetches) is 16 contiguous KB, so that weight streaming reads whole DRAM pages instead of
    128-byte pieces 2K bytes apart."""

    def __init__(self, w: torch.Tensor, swizzle: bool = False):
        N, K = w.shape
        assert N % 128 == 0 and K % 64 == 0, "tiled weights need N % 128 == 0 and K % 64 == 0"
        self.N, self.K = N, K
        self.swizzled = swizzle
        t = w.view(N // 128, 128, K // 64, 64).permute(0, 2, 1, 3).contiguous()
        if swizzle:  # the 128B-swizzle shared-memory image: 16-byte chunk c of row r sits at chunk c ^ (r % 8)
            r = torch.arange(128, device=w.device).view(128, 1)
            c = torch.arange(8, device=w.device).view(1, 8)
            idx = (c ^ (r & 7)).view(1, 1, 128, 8, 1).expand(N // 128, K // 64, 128, 8, 8)
            t = t.view(N // 128, K // 64, 128, 8, 8).gather(3, idx).contiguous()
        self.data = t.view(-1, 64)
        self.shape = (N, K)
        self.dtype, self.device = w.dtype, w.device

    def dense(self) -> torch.Tensor:
        N, K = self.N, self.K
        assert not self.swizzled
        return self.data.view(N // 128, K // 64, 128, 64).permute(0, 2, 1, 3).reshape(N, K)


_autotuner = None


def _tuned_bn(M: int, N: int, K: int, epi: str) -> int:
    global _autotuner
    if _autotuner is None:
        from ..utils import autotuner as _autotuner_mod

        _autotuner = _autotuner_mod
    return _autotuner.gemm_lookup(M, N, K, epi)


def gemm(a, w, epi: str = "store", residual=None, bias=None, out=None, bn: int = 0, stream_k: int = 0):
    """C = A . W^T on the tcgen05 tensor cores.  a [M, K], w [N, K] (checkpoint layout).

    epi: "store" | "residual" (C += residual) | "gated_silu"/"gated_gelu" (w rows interleaved with
    `reference.interleave_gate_up`, C is [M, N/2]) | "f32" (fp32 output, e.g. logits).
    stream_k: 0 whole tiles per CTA (default: fastest on every measured shape), 1 stream-K, -1 heuristic.
    """
    if type(w).__name__ == "Fp8Weight":  # block-scaled e4m3 weight: quantise the activations, fp8 tensor cores
        from . import fp8

        return fp8.gemm_fp8(a, w, epi, residual, bias, out)
    if type(w).__name__ == "Int8Weight":  # per-channel s8 weight, per-token s8 activations, s32 accumulation
        from . import int8

        return int8.gemm_int8(a, w, epi, residual, bias, out)
    if not _is_cuda(a):
        res = ref.gemm(a, w, epi, residual, bias)
        if out is not None:
            out.copy_(res)
            return out
        return res
    _req_bf16(a, w, residual, bias)
    if _GEMM_DEBUG_TORCH:  # debugging aid only (LLB_GEMM_DEBUG_TORCH=1): bypasses the tcgen05 kernel
        res = ref.gemm(a, w, epi, residual, bias)
        if out is not None:
            out.copy_(res)
            return out
        return res
    M, K = a.shape
    N = w.shape[0]
    tiled = isinstance(w, TiledWeight)
    if bn == 0 and stream_k == 0 and M <= 256 and bias is None and not tiled:  # a tuned variant, if one is stored
        bn = _tuned_bn(M, N, K, epi)
    ldw = (-2 if w.swizzled else -1) if tiled else w.stride(0)
    if tiled:
        w = w.data
    else:
        assert w.shape[1] == K and w.stride(1) == 1
    assert a.stride(1) == 1
    n_out = N // 2 if epi.startswith("gated") else N
    if out is None:
        out = torch.empty((M, n_out), dtype=torch.float32 if epi == "f32" else a.dtype, device=a.device)
    if epi == "residual":
        assert residual.shape == out.shape and residual.stride(0) == out.stride(0)
    skp, skc = (None, None) if (stream_k == 0 and not 2000 <= bn < 3100) else _stream_k_scratch(a.device)
    check(kernels().llb_gemm_bf16(ptr(a), i64(a.stride(0)), ptr(w), i64(ldw), ptr(out), i64(out.stride(0)),
                                  ptr(residual), ptr(bias), c_int(M), c_int(N), c_int(K), c_int(EPI_CODES[epi]),
                                  c_int(bn), c_int(stream_k), ptr(skp), i64(skp.numel() if skp is not None else 0),
                                  ptr(skc), c_int(skc.numel() if skc is not None else 0),
                                  ptr(gemm_status(a.device)), stream()), "gemm_bf16")
    _count()
    return out


# --------------------------------------------------------------------------------------
_decode_scratch = {}


def _scratch(device, n_o: int, n_lse: int):
    key = torch.device(device).index or 0
    cur = _decode_scratch.get(key)
    if cur is None or cur[0].numel() < n_o or cur[1].numel() < n_lse:
        cur = (torch.empty(max(n_o, 1 << 20), dtype=torch.float32, device=device),
               torch.empty(max(n_lse, 1 << 14), dtype=torch.float32, device=device))
        _decode_scratch[key] = cur
    return cur


def gqa_decode_num_splits(B, Hq, Hkv, max_seq_len) -> int:
    return int(kernels().llb_gqa_decode_num_splits(c_int(B), c_int(Hq), c_int(Hkv), c_int(max_seq_len)))


def gqa_decode(q, kv_layer, req_to_token, b_req_idx, b_seq_len, Hq, Hkv, D, max_seq_len: int, sm_scale=None,
               out=None, num_splits: Optional[int] = None, scratch=None):
    """Paged GQA decode attention. q [B, Hq*D] or [B, Hq, D] (row stride arbitrary)."""
    if isinstance(kv_layer, kv_quant.QuantKVLayer):
        return kv_quant.gqa_decode(q, kv_layer, req_to_token, b_req_idx, b_seq_len, Hq, Hkv, D, max_seq_len, sm_scale,
                                   out, num_splits, scratch)
    if not _is_cuda(q):
        return ref.gqa_decode(q.reshape(q.shape[0], Hq, D), kv_layer, req_to_token, b_req_idx, b_seq_len, Hq, Hkv, D,
                              sm_scale)
    _req_bf16(q, kv_layer)
    B = q.shape[0]
    assert q.stride(-1) == 1 and kv_layer.is_contiguous()
    assert req_to_token.dtype == torch.int32 and b_req_idx.dtype == torch.int32 and b_seq_len.dtype == torch.int32
    scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty((B, Hq, D), dtype=q.dtype, device=q.device)
    if num_splits is None:
        num_splits = gqa_decode_num_splits(B, Hq, Hkv, max_seq_len)
    po = pl = None
    if num_splits > 1:
        po, pl = scratch if scratch is not None else _scratch(q.device, B * Hq * num_splits * D, B * Hq * num_splits)
    check(kernels().llb_gqa_decode(ptr(q), i64(q.stride(0)), ptr(kv_layer), ptr(req_to_token),
                                   i64(req_to_token.stride(0)), ptr(b_req_idx), ptr(b_seq_len), ptr(out),
                                   i64(out.stride(0)), ptr(po), ptr(pl), c_int(B), c_int(Hq), c_int(Hkv), c_int(D),
                                   c_int(num_splits), f32(scale), stream()), "gqa_decode")
    _count(2 if num_splits > 1 else 1)
    return out


def gqa_prefill(q, kv_layer, req_to_token, b_req_idx, cu_q, b_ready_len, Hq, Hkv, D, max_q_len: int, sm_scale=None,
                out=None):
    """Causal varlen prefill attention over (cached prefix + new tokens). q [T, Hq*D] or [T, Hq, D]."""
    if isinstance(kv_layer, kv_quant.QuantKVLayer):
        return kv_quant.gqa_prefill(q, kv_layer, req_to_token, b_req_idx, cu_q, b_ready_len, Hq, Hkv, D, max_q_len,
                                    sm_scale, out)
    if not _is_cuda(q):
        return ref.gqa_prefill(q.reshape(q.shape[0], Hq, D), kv_layer, req_to_token, b_req_idx, cu_q, b_ready_len, Hq,
                               Hkv, D, sm_scale)
    _req_bf16(q, kv_layer)
    T = q.shape[0]
    B = b_req_idx.shape[0]
    assert q.stride(-1) == 1 and kv_layer.is_contiguous()
    assert cu_q.dtype == torch.int32 and b_ready_len.dtype == torch.int32
    scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty((T, Hq, D), dtype=q.dtype, device=q.device)
    check(kernels().llb_gqa_prefill(ptr(q), i64(q.stride(0)), ptr(kv_layer), ptr(req_to_token),
                                    i64(req_to_token.stride(0)), ptr(b_req_idx), ptr(cu_q), ptr(b_ready_len),
                                    ptr(out), i64(out.stride(0)), c_int(B), c_int(max_q_len), c_int(Hq), c_int(Hkv),
                                    c_int(D), f32(scale), stream()), "gqa_prefill")
    _count()
    return out


# --------------------------------------------------------------------------------------
def decode_prologue(req_to_token, next_token, b_req_idx, b_seq_len, new_slot, ids_out=None, pos_out=None):
    """ids[b] = next_token[req]; pos[b] = seq_len-1; req_to_token[req, seq_len-1] = new_slot[b]."""
    B = b_req_idx.shape[0]
    dev = b_req_idx.device
    if ids_out is None:
        ids_out = torch.empty(B, dtype=torch.int64, device=dev)
    if pos_out is None:
        pos_out = torch.empty(B, dtype=torch.int32, device=dev)
    if not b_req_idx.is_cuda:
        r = b_req_idx.long()
        ids_out.copy_(next_token[r, 0] if next_token.dim() == 2 else next_token[r])
        pos_out.copy_(b_seq_len - 1)
        req_to_token[r, (b_seq_len - 1).long()] = new_slot
        return ids_out, pos_out
    nt_stride = next_token.stride(0)
    check(kernels().llb_decode_prologue(ptr(ids_out), ptr(pos_out), ptr(req_to_token), ptr(next_token),
                                        ptr(b_req_idx), ptr(b_seq_len), ptr(new_slot), c_int(B),
                                        i64(req_to_token.stride(0)), c_int(nt_stride), stream()), "decode_prologue")
    _count()
    return ids_out, pos_out


def prefill_prologue(req_to_token, b_req_idx, b_ready_len, cu_q, new_slot, total_tokens: int):
    """positions / batch index of every new token and the slot table update, one launch."""
    dev = b_req_idx.device
    pos = torch.empty(total_tokens, dtype=torch.int32, device=dev)
    batch_of = torch.empty(total_tokens, dtype=torch.int32, device=dev)
    B = b_req_idx.shape[0]
    if not b_req_idx.is_cuda:
        for b in range(B):
            s, e = int(cu_q[b]), int(cu_q[b + 1])
            r = int(b_ready_len[b])
            pos[s:e] = torch.arange(r, r + e - s, dtype=torch.int32)
            batch_of[s:e] = b
            req_to_token[int(b_req_idx[b]), r:r + e - s] = new_slot[s:e]
        return pos, batch_of
    check(kernels().llb_prefill_prologue(ptr(pos), ptr(batch_of), ptr(req_to_token), ptr(b_req_idx), ptr(b_ready_len),
                                         ptr(cu_q), ptr(new_slot), c_int(B), i64(req_to_token.stride(0)), stream()),
          "prefill_prologue")
    _count()
    return pos, batch_of


def scatter_next_token_(next_token, sampled, b_req_idx, has_out=None):
    if not sampled.is_cuda:
        r = b_req_idx.long()
        if has_out is not None:
            m = has_out.bool()
            r, sampled = r[m], sampled[m]
        if next_token.dim() == 2:
            next_token[r, 0] = sampled
        else:
            next_token[r] = sampled
        return next_token
    B = sampled.shape[0]
    check(kernels().llb_scatter_next_token(ptr(next_token), ptr(sampled), ptr(b_req_idx), ptr(has_out), c_int(B),
                                           c_int(next_token.stride(0)), stream()), "scatter_next_token")
    _count()
    return next_token


def copy_rows(dst, src, dst_idx=None, src_idx=None, n_rows: Optional[int] = None):
    """dst[dst_idx[i]] = src[src_idx[i]] over rows (first dim); pinned host tensors allowed on either side."""
    if n_rows is None:
        n_rows = (dst_idx if dst_idx is not None else src_idx if src_idx is not None else src).shape[0]
    on_gpu = dst.is_cuda or src.is_cuda
    if not on_gpu:
        di = dst_idx.long() if dst_idx is not None else torch.arange(n_rows)
        si = src_idx.long() if src_idx is not None else torch.arange(n_rows)
        dst[di] = src[si]
        return dst
    row_bytes = src[0].numel() * src.element_size()
    check(kernels().llb_copy_rows(ptr(dst), ptr(src), ptr(dst_idx), ptr(src_idx), c_int(n_rows), i64(row_bytes),
                                  i64(dst.stride(0) * dst.element_size()), i64(src.stride(0) * src.element_size()),
                                  stream()), "copy_rows")
    _count()
    return dst


# --------------------------------------------------------------------------------------
def apply_penalty_(logits, presence, frequency, repetition, cu, tok_ids, tok_cnt, mask_cu=None, mask_ids=None):
    if not logits.is_cuda:
        return ref.apply_penalty_(logits, presence, frequency, repetition, cu, tok_ids, tok_cnt, mask_cu, mask_ids)
    assert logits.dtype == torch.float32
    B, V = logits.shape
    check(kernels().llb_apply_penalty(ptr(logits), i64(logits.stride(0)), ptr(presence), ptr(frequency),
                                      ptr(repetition), ptr(cu), ptr(tok_ids), ptr(tok_cnt), ptr(mask_cu),
                                      ptr(mask_ids), c_int(B), c_int(V), stream()), "apply_penalty")
    _count()
    return logits


def greedy_partials(logits, idx_off: int = 0):
    """First pass of the all-greedy sampler over (a vocabulary shard of) the logits: [B, S, 3] fp32 rows of
    (max, arg-max as global token id bits, sum exp(x - max)).  S depends on B and the shard width only."""
    B, V = logits.shape
    splits = max(1, min(64, 2368 // max(B, 1), V // 2048))
    if not logits.is_cuda:
        return ref.greedy_partials(logits, idx_off, splits)
    dt = {torch.float32: 0, torch.bfloat16: 1}[logits.dtype]
    part = torch.empty((B, splits, 3), dtype=torch.float32, device=logits.device)
    check(kernels().llb_greedy_partial(ptr(logits), c_int(dt), i64(logits.stride(0)), c_int(B), c_int(V),
                                       c_int(idx_off), ptr(part), c_int(splits), stream()), "greedy_partial")
    _count()
    return part


def greedy_merge(parts):
    """parts [R, B, S, 3] (the partials of R vocabulary shards) -> (ids int64 [B], logprob fp32 [B])."""
    R, B, S, _ = parts.shape
    if not parts.is_cuda:
        return ref.greedy_merge(parts)
    parts = parts.contiguous()
    ids = torch.empty(B, dtype=torch.int64, device=parts.device)
    lp = torch.empty(B, dtype=torch.float32, device=parts.device)
    check(kernels().llb_greedy_merge(ptr(parts), c_int(B), c_int(S), c_int(R), ptr(ids), ptr(lp), stream()),
          "greedy_merge")
    _count()
    return ids, lp


def sample(logits, temperature=None, top_p=None, top_k=None, seeds=None, steps=None, want_logprob=True):
    """Returns (ids int64 [B], logprob fp32 [B]).  Rows with top_k == 1 (or top_k None) are greedy.
    `logits` may be vocabulary-parallel (`common.infer_state.ShardedLogits`): an all-greedy batch is then
    sampled from the shards (a few KB exchanged per step), anything else from the gathered matrix."""
    if hasattr(logits, "greedy"):
        if temperature is None and top_k is None and top_p is None:
            return logits.greedy()
        logits = logits.full()
    if not logits.is_cuda:
        return ref.sample(logits, temperature, top_p, top_k, seeds, steps)
    B, V = logits.shape
    dt = {torch.float32: 0, torch.bfloat16: 1}[logits.dtype]
    ids = torch.empty(B, dtype=torch.int64, device=logits.device)
    lp = torch.empty(B, dtype=torch.float32, device=logits.device) if want_logprob else None
    if temperature is None and top_k is None and top_p is None:  # every row greedy: many CTAs per row
        splits = max(1, min(64, 2368 // B, V // 2048))
        scratch = torch.empty(B * splits * 3, dtype=torch.float32, device=logits.device)
        check(kernels().llb_sample_greedy(ptr(logits), c_int(dt), i64(logits.stride(0)), c_int(B), c_int(V), ptr(scratch),
                                          c_int(splits), ptr(ids), ptr(lp), stream()), "sample_greedy")
        _count(2)
        return ids, lp
    if seeds is not None:
        assert seeds.dtype == torch.int64
    check(kernels().llb_sample(ptr(logits), c_int(dt), i64(logits.stride(0)), c_int(B), c_int(V), ptr(temperature),
                               ptr(top_p), ptr(top_k), ptr(seeds), ptr(steps), ptr(ids), ptr(lp), stream()), "sample")
    _count()
    return ids, lp


def token_logprob(logits, ids):
    if not logits.is_cuda:
        return ref.token_logprob(logits, ids)
    B, V = logits.shape
    dt = {torch.float32: 0, torch.bfloat16: 1}[logits.dtype]
    out = torch.empty(B, dtype=torch.float32, device=logits.device)
    check(kernels().llb_token_logprob(ptr(logits), c_int(dt), i64(logits.stride(0)), c_int(B), c_int(V), ptr(ids),
                                      ptr(out), stream()), "token_logprob")
    _count()
    return out


# --------------------------------------------------------------------------------------
def layernorm(x, w, b, eps: float, residual=None):
    """LayerNorm(x [+ residual]) * w + b; with `residual` the sum is written back into it (in place)."""
    if not _is_cuda(x):
        return ref.layernorm(x, w, b, eps, residual)
    _req_bf16(x, w)
    assert x.is_contiguous() and (residual is None or residual.is_contiguous())
    T, H = x.shape
    out = torch.empty_like(x)
    check(kernels().llb_layernorm(ptr(out), ptr(residual), ptr(x), ptr(w), ptr(b), c_int(T), c_int(H), f32(eps),
                                  stream()), "layernorm")
    _count()
    return out


def act_(x, kind: str, alpha: float = 1.0):
    """In-place activation (silu | gelu | gelu_tanh | relu) or scaling (kind "scale", factor alpha)."""
    if not _is_cuda(x):
        return ref.act_(x, kind, alpha)
    _req_bf16(x)
    assert x.is_contiguous()
    check(kernels().llb_act_(ptr(x), i64(x.numel()), c_int(ref.ACT_KINDS[kind]), f32(alpha), stream()), "act")
    _count()
    return x


def attention_generic(q, kv_layer, req_to_token, b_req_idx, pos, batch_of, Hq, Hkv, D, sm_scale, window: int = 0,
                      softcap: float = 0.0, alibi=None, sinks=None):
    """Causal paged attention for any head size <= 256 with sliding window / ALiBi / soft-cap / sinks.
    q [T, Hq*D] or [T, Hq, D]; returns [T, Hq, D]."""
    T = q.shape[0]
    if isinstance(kv_layer, kv_quant.QuantKVLayer):
        return kv_quant.attention_generic(q, kv_layer, req_to_token, b_req_idx, pos, batch_of, Hq, Hkv, D, sm_scale,
                                          window, softcap, alibi, sinks)
    if not _is_cuda(q):
        return ref.attention_generic(q.reshape(T, Hq, D), kv_layer, req_to_token, b_req_idx, pos, batch_of, Hq, Hkv, D,
                                     sm_scale, window, softcap, alibi, sinks)
    _req_bf16(q, kv_layer)
    assert q.stride(-1) == 1 and kv_layer.is_contiguous() and pos.dtype == torch.int32
    out = torch.empty((T, Hq, D), dtype=q.dtype, device=q.device)
    check(kernels().llb_attn_generic(ptr(q), i64(q.stride(0)), ptr(kv_layer), ptr(req_to_token),
                                     i64(req_to_token.stride(0)), ptr(b_req_idx), ptr(pos), ptr(batch_of), ptr(out),
                                     i64(out.stride(0)), c_int(T), c_int(Hq), c_int(Hkv), c_int(D), f32(sm_scale),
                                     c_int(window), f32(softcap), ptr(alibi), ptr(sinks), stream()), "attn_generic")
    _count()
    return out
