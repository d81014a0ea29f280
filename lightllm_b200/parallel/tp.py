"""Tensor-parallel communication used by the layers.

The layer code asks for *semantics* ("reduce the row-parallel partial sums, add the residual,
normalise for the next block"); this object picks the implementation:

  * tp == 1            : nothing to reduce (the GEMM epilogue already added the residual)
  * fused (CUDA, NVLink): one kernel of `parallel.fused` does reduce + residual + RMSNorm over
                          peer memory (one-shot for decode-sized messages, two-shot otherwise)
  * baseline            : torch.distributed all-reduce (NCCL / gloo) followed by add_rmsnorm_

Reference behaviour: lightllm/common/basemodel/layer_infer/base_layer_infer.py:53-98 (all-reduce
or reduce-scatter/all-gather in TPSP mode) with separate add and rmsnorm kernels.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from . import dist as pdist


class TPContext:
    def __init__(self, pstate: Optional[pdist.ParallelState] = None, fused=None):
        st = pstate or pdist.state()
        self.size = st.tp_size
        self.rank = st.tp_rank
        self.group = st.tp_group
        self.device = st.device
        self.fused = fused  # parallel.fused.FusedTP or None
        self.ce = None      # parallel.ce.CopyEngineTP (pipelined prompt passes), attached after the model is built

    # ---- primitives ----
    def all_reduce_(self, x):
        if self.size == 1:
            return x
        # plain all-reduces (vocabulary-parallel embedding, the last layer's partial sums) are rare per pass:
        # they stay on the library collective; the fused kernels cover reduce + residual + norm
        dist.all_reduce(x, group=self.group)
        return x

    def all_gather_rows(self, x):
        """[n, ...] per rank -> [tp*n, ...]."""
        if self.size == 1:
            return x
        out = torch.empty((self.size * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def gather_logits(self, local_logits):
        """[B, V/tp] per rank -> [B, V] (vocab-parallel lm_head)."""
        if self.size == 1:
            return local_logits
        B, Vl = local_logits.shape
        out = torch.empty((self.size * B, Vl), dtype=local_logits.dtype, device=local_logits.device)
        dist.all_gather_into_tensor(out, local_logits.contiguous(), group=self.group)
        return out.view(self.size, B, Vl).permute(1, 0, 2).reshape(B, self.size * Vl)

    # ---- fused semantics ----
    def reduce_residual_norm(self, partial, residual, norm_w, eps, w_offset=0.0):
        """residual += sum_over_ranks(partial); returns rmsnorm(residual) * norm_w."""
        if self.size > 1:
            if self.fused is not None and self.fused.owns(partial):
                return self.fused.reduce_residual_norm(partial, residual, norm_w, eps, w_offset)
            self.all_reduce_(partial)
        return ops.add_rmsnorm_(residual, partial, norm_w, eps, w_offset)
