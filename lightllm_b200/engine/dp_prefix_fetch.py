"""Cross-replica prefix fetch for data-parallel serving (`--enable_dp_prompt_cache_fetch`).

Every replica keeps its own KV pool and prefix tree.  When a new request is assigned to replica A although replica B
holds a longer cached prefix of its prompt, A copies the missing KV rows from B instead of recomputing them.  All
ranks see the same batch of new requests at the same point of their loops (the router's message), so the exchange is
a collective phase:

  1. every rank looks the prompts up in its own tree (read-only; the matched nodes are pinned for the duration);
  2. one host all-gather of (match lengths, free tokens) gives every rank the same picture; the same plan is computed
     everywhere: per request the lowest replica with the longest match is the source if it beats the owner's own
     match by at least `min_gain` tokens and the owner has room;
  3. per planned copy, rank (source replica, t) gathers the rows of its KV shard into a staging buffer and sends
     them to rank (owner replica, t); the receiver scatters them into fresh slots and publishes them in its prefix
     tree, where the normal admission finds them.  Rows are opaque pool rows, so every pool type works.

Reference: lightllm/server/router/model_infer/mode_backend/dp_backend/dp_shared_kv_trans.py:1-139 (same decision
rule; it reads the other replica's pool through CUDA IPC mappings of all pools in the node, here the rows travel by
point-to-point send / recv of the device process group, NCCL over NVLink on GPUs).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist


def plan_fetches(match: np.ndarray, owners: Sequence[int], prompt_lens: Sequence[int], free: np.ndarray,
                 min_gain: int = 32) -> List[Tuple[int, int, int, int, int]]:
    """match [replicas, requests] (tokens each replica has cached of each prompt), owners[request], free[replica].
    Returns (request, source replica, owner, start, end) copies, identical on every rank."""
    free = np.array(free, dtype=np.int64).copy()
    plan = []
    for j, owner in enumerate(owners):
        col = match[:, j]
        src = int(np.argmax(col))                  # lowest replica among the longest matches
        end = min(int(col[src]), int(prompt_lens[j]) - 1)   # the last prompt token always runs through the model
        start = int(col[owner])
        n = end - start
        if src == owner or n < min_gain or free[owner] <= n:
            continue
        free[owner] -= n
        plan.append((j, src, int(owner), start, end))
    return plan


class DPPrefixFetch:
    def __init__(self, backend, min_gain: int = 32, chunk_tokens: int = 4096):
        self.b = backend
        self.ps = backend.model.ps
        self.min_gain, self.chunk = min_gain, chunk_tokens
        self.stats = {"fetched_tokens": 0, "served_tokens": 0, "rounds": 0}

    def run(self, new_reqs: Sequence[Tuple[int, np.ndarray]]) -> int:
        """`new_reqs`: (owner replica, prompt token ids) of EVERY new request of this round, the same list on every
        rank.  Collective over all ranks.  Returns the number of tokens this rank received."""
        ps, ctx = self.ps, self.b.ctx
        cache, mm = ctx.radix_cache, ctx.mem_manager
        if ps.dp_size <= 1 or cache is None or not new_reqs:
            return 0
        self.stats["rounds"] += 1
        n = len(new_reqs)
        mine = torch.zeros(n + 1, dtype=torch.int64)
        held = []
        for j, (_, ids) in enumerate(new_reqs):
            node, m, slots = cache.match_prefix(np.asarray(ids[:-1], dtype=np.int64), update_refs=True)
            held.append((node, slots))
            mine[j] = m
        mine[n] = ctx.get_can_alloc_token_num()
        allv = torch.empty(ps.world_size * (n + 1), dtype=torch.int64)
        dist.all_gather_into_tensor(allv, mine, group=ps.cpu_group)
        allv = allv.view(ps.world_size, n + 1).numpy()
        per_replica = allv[::ps.tp_size]          # ranks of a replica hold the same tree: take its first rank
        plan = plan_fetches(per_replica[:, :n], [o for o, _ in new_reqs], [len(i) for _, i in new_reqs],
                            per_replica[:, n], self.min_gain)
        got = 0
        try:
            for j, src, owner, start, end in plan:
                ids = np.asarray(new_reqs[j][1], dtype=np.int64)
                if ps.dp_rank == src:
                    self._send(held[j][1][start:end], owner * ps.tp_size + ps.tp_rank)
                    self.stats["served_tokens"] += end - start
                elif ps.dp_rank == owner:
                    got += self._recv(ids, held[j], start, end, src * ps.tp_size + ps.tp_rank)
        finally:
            for node, _ in held:
                if node is not None:
                    cache.dec_node_ref_counter(node)
        self.stats["fetched_tokens"] += got
        return got

    # ------------------------------------------------------------------
    def _send(self, slots: np.ndarray, dst_rank: int):
        mm = self.b.ctx.mem_manager
        for a in range(0, len(slots), self.chunk):
            pages = mm.gather_pages(torch.from_numpy(np.ascontiguousarray(slots[a:a + self.chunk])).to(torch.int32))
            dist.send(pages.view(torch.uint8).contiguous() if pages.dtype not in (torch.uint8, torch.int8)
                      else pages.contiguous(), dst=dst_rank)

    def _recv(self, ids: np.ndarray, held, start: int, end: int, src_rank: int) -> int:
        ctx = self.b.ctx
        mm, cache = ctx.mem_manager, ctx.radix_cache
        n = end - start
        new_slots = ctx.alloc_slots(n)
        for a in range(0, n, self.chunk):
            m = min(self.chunk, n - a)
            pages = torch.empty((mm.layer_num, m, *mm.kv_row_shape()), dtype=mm.dtype, device=mm.device)
            wire = pages.view(torch.uint8) if pages.dtype not in (torch.uint8, torch.int8) else pages
            dist.recv(wire, src=src_rank)
            mm.scatter_pages(new_slots[a:a + m], pages)
        # key = the prompt up to `end`; the first `start` positions are already in the tree (their slots are
        # repeated here and, being present, are ignored by the insert)
        own = held[1][:start] if start > 0 else np.zeros(0, dtype=np.int32)
        value = np.concatenate([np.asarray(own, dtype=np.int32), new_slots.cpu().numpy().astype(np.int32)])
        present = cache.insert(ids[:end], value)
        if present > start:      # somebody published part of it meanwhile: the spare copies go back to the pool
            mm.free(value[start:present])
        return n
