"""Token re-balancing of prompt passes across data-parallel replicas (`--enable_dp_prefill_balance`).

Replicas step in lock-step, so a prompt pass takes as long as the replica with the most tokens needs.  Everything in
a decoder layer except the attention itself is token-wise (projections, router, shared and routed experts, norms),
so those parts can run on an even split of all replicas' tokens: the embeddings are exchanged into the balanced
layout once, each layer brings the normalised stream back to the owners for the attention block (which needs the
owner's KV pool) and its output forth again, and the final hidden states return to their owners for the logits.

The exchange is one variable-size all-to-all over the group of equal tensor-parallel ranks of all replicas; the
split sizes are computed by every rank from an all-gather of the token counts: every replica keeps as many of its
own tokens as its even share allows, the surplus of the loaded replicas fills the others in rank order.

Reference: lightllm/common/basemodel/infer_struct.py:167-351 (prepare_prefill_dp_balance and the two all-to-all
helpers; same even split).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def plan_balance(lens: List[int], multiple: int = 1) -> List[List[int]]:
    """S[s][d] = tokens of replica s handled by replica d.  Row sums are `lens`, column sums the even shares
    (in units of `multiple` tokens)."""
    n = len(lens)
    assert all(x % multiple == 0 for x in lens)
    units = [x // multiple for x in lens]
    total = sum(units)
    share = [total // n + (1 if i < total % n else 0) for i in range(n)]
    S = [[0] * n for _ in range(n)]
    surplus, need = [], []
    for i in range(n):
        keep = min(units[i], share[i])
        S[i][i] = keep
        if units[i] > keep:
            surplus.append([i, units[i] - keep])
        if share[i] > keep:
            need.append([i, share[i] - keep])
    si = 0
    for d, want in need:
        while want > 0:
            s, have = surplus[si]
            take = min(have, want)
            S[s][d] += take
            want -= take
            surplus[si][1] -= take
            if surplus[si][1] == 0:
                si += 1
    return [[v * multiple for v in row] for row in S]


class DPBalance:
    """The exchange of one prompt pass.  `to_balanced(x)`: rows of my own tokens -> rows of the tokens I handle;
    `to_origin(y)` is its inverse."""

    def __init__(self, S: List[List[int]], me: int, group):
        self.S, self.me, self.group = S, me, group
        self.send = [S[me][d] for d in range(len(S))]          # my tokens, dealt to the replicas in rank order
        self.recv = [S[s][me] for s in range(len(S))]
        self.origin_len, self.handle_len = sum(self.send), sum(self.recv)

    @classmethod
    def prepare(cls, ps, my_tokens: int, min_gain: float = 0.1) -> Optional["DPBalance"]:
        """Collective over all ranks.  None when the pass is balanced enough already (the largest replica would
        shed less than `min_gain` of its tokens)."""
        mine = torch.tensor([my_tokens], dtype=torch.int64)
        allv = torch.empty(ps.world_size, dtype=torch.int64)
        dist.all_gather_into_tensor(allv, mine, group=ps.cpu_group)
        lens = allv[::ps.tp_size].tolist()
        top = max(lens)
        share = -(-sum(lens) // len(lens))
        if top == 0 or top - share < min_gain * top:
            return None
        return cls(plan_balance(lens), ps.dp_rank, ps.dp_peer_group)

    def _exchange(self, x: torch.Tensor, n_out: int, out_split, in_split) -> torch.Tensor:
        x = x.contiguous()
        out = torch.empty((n_out, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x, output_split_sizes=list(out_split), input_split_sizes=list(in_split),
                               group=self.group)
        return out

    def to_balanced(self, x: torch.Tensor) -> torch.Tensor:
        assert x.shape[0] == self.origin_len
        return self._exchange(x, self.handle_len, self.recv, self.send)

    def to_origin(self, y: torch.Tensor) -> torch.Tensor:
        assert y.shape[0] == self.handle_len
        return self._exchange(y, self.origin_len, self.send, self.recv)
