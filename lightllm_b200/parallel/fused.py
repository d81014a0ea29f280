"""Fused tensor-parallel reduction: all-reduce over NVLink peer memory + residual add + RMSNorm in
one kernel (`csrc/comm.cu`), used after every row-parallel GEMM.

The row-parallel GEMM writes its partial sums straight into this rank's symmetric `partial` buffer
(`partial_out(T)` hands out the view for the current call), then `reduce_residual_norm` launches the
kernel.  Two buffers alternate between calls; every forward pass issues an even number of calls (two per
layer), so the buffer a call site uses is the same on every CUDA-graph replay.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..ops import _count
from ..ops._native import check, f32, kernels, ptr, stream
from . import dist as pdist
from .symm import SymmetricRegion


def _ptr_array(vals):
    arr = (ctypes.c_void_p * len(vals))()
    for i, v in enumerate(vals):
        arr[i] = v
    return arr


class FusedTP:
    ONE_SHOT_BYTES = 512 * 1024  # per-rank message below which every rank pulls all rows itself

    def __init__(self, pstate: Optional[pdist.ParallelState] = None, max_tokens: int = 16384, hidden: int = 8192,
                 ctas: int = 64):
        ps = pstate or pdist.state()
        assert ps.device.type == "cuda" and 1 < ps.tp_size <= 8
        self.ps = ps
        self.world, self.rank = ps.tp_size, ps.tp_rank
        self.max_tokens, self.hidden = max_tokens, hidden
        self.ctas = ctas
        row_bytes = hidden * 2
        self.buf_bytes = ((max_tokens * row_bytes + 255) // 256) * 256
        self.off_partial = [0, self.buf_bytes]
        self.off_sums = [2 * self.buf_bytes, 3 * self.buf_bytes]
        self.off_ready = 4 * self.buf_bytes
        self.off_rowflag = self.off_ready + 256
        total = self.off_rowflag + ((max_tokens * 4 + 255) // 256) * 256
        group = ps.cpu_group if ps.cpu_group is not None else ps.tp_group
        self.region = SymmetricRegion(total, self.rank, self.world, group=ps.tp_group if ps.dp_size > 1 else group,
                                      device=ps.device)
        self.local = torch.zeros(4, dtype=torch.int32, device=ps.device)  # [epoch, arrive, status, pad]
        self.parity = 0
        self.calls = 0

    # ---- buffers ----
    def partial_out(self, T: int, H: int) -> torch.Tensor:
        """Where the row-parallel GEMM of the next call must write its [T, H] partial sums."""
        assert T <= self.max_tokens and H == self.hidden
        return self.region.tensor(self.off_partial[self.parity], (T, H), torch.bfloat16)

    def owns(self, partial) -> bool:
        """True if `partial` is the buffer handed out by `partial_out` for the coming call."""
        return partial.is_cuda and partial.data_ptr() == self.region.local_ptr + self.off_partial[self.parity]

    def can_all_reduce(self, x) -> bool:
        return False  # plain all-reduces (embedding, final residual) stay on NCCL

    def _launch(self, T, H, residual, out, norm_w, eps, w_offset, do_norm):
        r = self.region
        par = self.parity
        one_shot = 1 if T * H * 2 <= self.ONE_SHOT_BYTES else 0
        partial = _ptr_array([r.ptrs[q] + self.off_partial[par] for q in range(self.world)])
        sums = _ptr_array([r.ptrs[q] + self.off_sums[par] for q in range(self.world)])
        ready = _ptr_array([r.ptrs[q] + self.off_ready for q in range(self.world)])
        rowflag = _ptr_array([r.ptrs[q] + self.off_rowflag for q in range(self.world)])
        base = self.local.data_ptr()
        check(kernels().llb_tp_reduce_norm(partial, sums, ready, rowflag, _ptr_array([residual.data_ptr() if residual is not None else 0]),
                                           _ptr_array([out.data_ptr()]), ptr(norm_w), _ptr_array([base]),
                                           _ptr_array([base + 4]), ctypes.c_void_p(base + 8), ctypes.c_int(self.rank),
                                           ctypes.c_int(self.world), ctypes.c_int(0), ctypes.c_int(T), ctypes.c_int(H),
                                           f32(eps), f32(w_offset), ctypes.c_int(one_shot), ctypes.c_int(do_norm),
                                           ctypes.c_int(min(self.ctas, max(T, 1))), stream()), "tp_reduce_norm")
        _count()
        self.parity ^= 1
        self.calls += 1

    def reduce_residual_norm(self, partial, residual, norm_w, eps, w_offset=0.0):
        """`partial` must be the tensor handed out by `partial_out` for this call."""
        T, H = partial.shape
        assert partial.data_ptr() == self.region.local_ptr + self.off_partial[self.parity], \
            "the row-parallel GEMM must write into FusedTP.partial_out()"
        out = torch.empty((T, H), dtype=torch.bfloat16, device=partial.device)
        self._launch(T, H, residual, out, norm_w, eps, w_offset, 1)
        return out

    def all_reduce_(self, x):
        raise NotImplementedError

    def status(self) -> int:
        return int(self.local[2].item())
