"""Prompt-sized tensor-parallel reduction on the copy engines.

After a row-parallel GEMM (o_proj, down_proj) of a prompt pass every rank holds [T, H] partial sums.  This module
turns them into the normalised input of the next block in the token-sharded form (reduce-scatter, residual add and
RMSNorm on the rows a rank owns, all-gather of the normalised rows; the reference's tpsp mix mode,
lightllm/common/basemodel/layer_infer/base_layer_infer.py:63-98, does the same with NCCL reduce-scatter /
all-gather and separate add / norm kernels), with the wire traffic carried by stream-ordered peer copies:

    flag exchange "partial of call e complete"       one 32-thread kernel
    pull my row slice of every peer's partial        world - 1 copies over NVLink, DMA engines
    sum + residual + RMSNorm on my rows              one small kernel
    flag exchange "my normalised rows are ready"
    pull every peer's normalised rows                world - 1 copies

No SM is busy while the bytes move, so a reduction issued on a side stream runs under the GEMMs and the attention
of another micro-batch (`TransformerLM._prefill_pipelined`), which NCCL's or this package's SM-resident reduction
kernels do not allow (they need their CTAs co-resident with a persistent GEMM that already fills every SM).

Buffers live in one symmetric region per rank: partial[2][max_tokens, H] (the GEMM writes into it), gather[2][...]
(normalised rows, every rank ends up with all of them) and two flag arrays.  Calls alternate between the two
halves.  A rank cannot finish call e before every peer has announced its normalised rows of call e, which a peer
does only after its own pulls of call e are done; hence when a rank reuses a half for call e + 2 nobody reads it
any more.  Flags carry the call number and only grow.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from ..ops import _count
from ..ops._native import check, f32, i64, kernels, ptr
from . import dist as pdist
from .fused import _ptr_array
from .symm import SymmetricRegion, view_device_memory


class CopyEngineTP:
    WAIT_MS = 8000

    def __init__(self, rank: int, world: int, max_tokens: int, hidden: int, device, ptrs: List[int], local_ptr: int,
                 region=None):
        assert hidden % 8 == 0
        self.rank, self.world, self.max_tokens, self.hidden = rank, world, max_tokens, hidden
        self.device = device
        self.region = region
        self.buf_bytes = self.layout(max_tokens, hidden)[0]
        self.off_partial = [0, self.buf_bytes]
        self.off_gather = [2 * self.buf_bytes, 3 * self.buf_bytes]
        self.off_ready = 4 * self.buf_bytes
        self.off_normed = self.off_ready + 256
        self.ptrs, self.local_ptr = list(ptrs), local_ptr
        self._bytes = view_device_memory(local_ptr, self.layout(max_tokens, hidden)[1], device)
        rows = (max_tokens + world - 1) // world
        self.stage = torch.empty((max(world - 1, 1), rows, hidden), dtype=torch.bfloat16, device=device)
        self.status_word = torch.zeros(1, dtype=torch.int32, device=device)
        self.calls = 0
        self._ready_tab = _ptr_array([p + self.off_ready for p in self.ptrs])
        self._normed_tab = _ptr_array([p + self.off_normed for p in self.ptrs])

    @staticmethod
    def layout(max_tokens: int, hidden: int):
        buf = ((max_tokens * hidden * 2 + 255) // 256) * 256
        return buf, 4 * buf + 512

    @classmethod
    def create(cls, pstate: Optional[pdist.ParallelState] = None, max_tokens: int = 16384, hidden: int = 4096):
        ps = pstate or pdist.state()
        assert ps.device.type == "cuda" and 1 < ps.tp_size <= 8
        total = cls.layout(max_tokens, hidden)[1]
        group = ps.cpu_group if ps.cpu_group is not None else ps.tp_group
        region = SymmetricRegion(total, ps.tp_rank, ps.tp_size, group=ps.tp_group if ps.dp_size > 1 else group,
                                 device=ps.device)
        return cls(ps.tp_rank, ps.tp_size, max_tokens, hidden, ps.device, region.ptrs, region.local_ptr, region)

    def close(self):
        self._bytes = None
        if self.region is not None:
            self.region.close()
            self.region = None

    # ---- views ----
    def _view(self, off: int, T: int) -> torch.Tensor:
        n = T * self.hidden * 2
        return self._bytes[off:off + n].view(torch.bfloat16).view(T, self.hidden)

    def partial_out(self, T: int) -> torch.Tensor:
        """Where the row-parallel GEMM of the next call must write its [T, H] partial sums."""
        assert T <= self.max_tokens
        return self._view(self.off_partial[self.calls & 1], T)

    def rows_of(self, q: int, T: int):
        per = (T + self.world - 1) // self.world
        return min(T, q * per), min(T, (q + 1) * per)

    def status(self) -> int:
        return int(self.status_word.item())

    # ---- the three phases of a call (run back to back by `reduce`; split for single-GPU emulation) ----
    def _signal_wait(self, tab, off, code, mode: int = 3):
        st = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        check(kernels().llb_ce_signal_wait(tab, ctypes.c_void_p(self.local_ptr + off), ctypes.c_int(self.rank),
                                           ctypes.c_int(self.world), ctypes.c_uint32(self.calls + 1),
                                           ptr(self.status_word), ctypes.c_int(code), i64(self.WAIT_MS), ctypes.c_int(mode), st),
              "ce_signal_wait")
        _count()

    def _copy(self, dst: int, src: int, nbytes: int):
        st = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        check(kernels().llb_memcpy_async(ctypes.c_void_p(dst), ctypes.c_void_p(src), i64(nbytes), st), "memcpy_async")

    def phase_ready(self, mode: int = 3):
        """mode: 1 announce only, 2 wait only, 3 both (single-GPU emulation runs the two halves separately)."""
        self._signal_wait(self._ready_tab, self.off_ready, 800, mode)

    def phase_scatter_reduce(self, T: int, residual, norm_w, eps: float, w_offset: float = 0.0):
        par, H = self.calls & 1, self.hidden
        lo, hi = self.rows_of(self.rank, T)
        n = hi - lo
        row_bytes = H * 2
        srcs = [self.local_ptr + self.off_partial[par] + lo * row_bytes]
        if n > 0:
            for i in range(1, self.world):
                q = (self.rank + i) % self.world        # every rank starts at another peer: the pulls spread out
                slot = self.stage[i - 1]
                self._copy(slot.data_ptr(), self.ptrs[q] + self.off_partial[par] + lo * row_bytes, n * row_bytes)
                srcs.append(slot.data_ptr())
            st = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
            check(kernels().llb_ce_reduce_norm(_ptr_array(srcs), ctypes.c_int(len(srcs)),
                                               ctypes.c_void_p(residual.data_ptr() + lo * row_bytes),
                                               ctypes.c_void_p(self.local_ptr + self.off_gather[par] + lo * row_bytes),
                                               ptr(norm_w), ctypes.c_int(n), ctypes.c_int(H), f32(eps), f32(w_offset),
                                               st), "ce_reduce_norm")
            _count()

    def phase_normed(self, mode: int = 3):
        self._signal_wait(self._normed_tab, self.off_normed, 810, mode)

    def phase_gather(self, T: int) -> torch.Tensor:
        par, row_bytes = self.calls & 1, self.hidden * 2
        for i in range(1, self.world):
            q = (self.rank + i) % self.world
            lo, hi = self.rows_of(q, T)
            if hi > lo:
                off = self.off_gather[par] + lo * row_bytes
                self._copy(self.local_ptr + off, self.ptrs[q] + off, (hi - lo) * row_bytes)
        out = self._view(self.off_gather[par], T)
        self.calls += 1
        return out

    def reduce(self, partial, residual, norm_w, eps: float, w_offset: float = 0.0) -> torch.Tensor:
        """`partial` must be the tensor handed out by `partial_out`.  residual[my rows] += sum over ranks; returns
        the complete normalised [T, H] activations (a view that stays valid until the call after the next one).
        Only this rank's rows of `residual` are kept up to date.  Everything is queued on the current stream."""
        T = partial.shape[0]
        assert partial.data_ptr() == self.local_ptr + self.off_partial[self.calls & 1], \
            "the row-parallel GEMM must write into CopyEngineTP.partial_out()"
        self.phase_ready()
        self.phase_scatter_reduce(T, residual, norm_w, eps, w_offset)
        self.phase_normed()
        return self.phase_gather(T)


    def self_test(self, group, T: int = 48) -> bool:
        """Two small reductions (both buffer halves) against NCCL + torch on the same numbers; every rank learns
        whether ALL ranks agreed, so that they take the same decision about using this path."""
        import torch.distributed as dist

        dev, H = self.device, self.hidden
        T = min(T, self.max_tokens)
        ok = True
        try:
            for k in range(2):
                g = torch.Generator(device=dev).manual_seed(977 + 31 * k + self.rank)
                mine = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
                gs = torch.Generator(device=dev).manual_seed(55 + k)
                residual = torch.randn(T, H, generator=gs, device=dev).to(torch.bfloat16)
                total = mine.float()
                dist.all_reduce(total, group=group)
                want_res = residual.float() + total
                want = want_res * torch.rsqrt(want_res.pow(2).mean(-1, keepdim=True) + 1e-6)
                partial = self.partial_out(T)
                partial.copy_(mine)
                res = residual.clone()
                got = self.reduce(partial, res, torch.ones(H, dtype=torch.bfloat16, device=dev), 1e-6)
                torch.cuda.synchronize(dev)
                lo, hi = self.rows_of(self.rank, T)
                ok = ok and self.status() == 0 and \
                    (got.float() - want).abs().max().item() < 0.05 * max(want.abs().max().item(), 1.0)
                if hi > lo:
                    scale = max(want_res.abs().max().item(), 1.0)
                    ok = ok and (res[lo:hi].float() - want_res[lo:hi]).abs().max().item() < 0.05 * scale
        except Exception:
            ok = False
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        return bool(flag.item())


def attach(model, pstate, max_tokens: int, log=print) -> bool:
    """Gives a tensor-parallel model on GPUs the copy-engine reducer its pipelined prompt passes use
    (LLB_PREFILL_PIPELINE=0 keeps the single-stream schedule).  Collective: every rank of the replica must call it."""
    import os

    if pstate.tp_size <= 1 or pstate.device.type != "cuda" or os.environ.get("LLB_PREFILL_PIPELINE", "1") == "0":
        return False
    ce = None
    try:
        ce = CopyEngineTP.create(pstate, max_tokens=max_tokens, hidden=model.hidden)
        ok = ce.self_test(pstate.tp_group)
    except Exception as e:  # noqa: BLE001
        ok = False
        if log:
            log(f"[rank {pstate.global_rank}] copy-engine reducer unavailable: {type(e).__name__}: {e}")
    if not ok:
        if ce is not None:
            ce.close()
        return False
    model.tp.ce = ce
    return True
