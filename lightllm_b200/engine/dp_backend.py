"""Data-parallel attention: every replica (a tensor-parallel group; a single rank when --dp equals the world
size) serves its own requests with its own KV pool and prefix tree, but all ranks of the world step together,
because the expert-parallel MoE layers exchange tokens between all of them.  Before each step the ranks
all-gather (prefill tokens, decode requests) on the host group: if anyone prefills, everybody runs a prefill
pass; else if anyone decodes, everybody decodes; a rank with nothing of that kind runs the pass on the HOLD
request (one dummy token, HOLD KV slot) so that it still takes part in the exchanges.
Reference: mode_backend/dp_backend/impl.py:97-152, base_backend.py:933-959.
"""
from __future__ import annotations

import time

import numpy as np
import torch
import torch.distributed as dist

from ..common.infer_state import ModelInput
from .backend import ModelBackend


class DPBackend(ModelBackend):
    def __init__(self, *a, idle_sleep_s: float = 0.001, **kw):
        super().__init__(*a, **kw)
        self.ps = self.model.ps
        self.idle_sleep_s = idle_sleep_s
        self.stats.update({"hold_prefill": 0, "hold_decode": 0})
        self.redundancy = None    # re-places this rank's redundant expert copies from live hit counters
        if self.model.extra.get("auto_update_redundancy_expert") and \
                any(getattr(lw, "ep_table", None) is not None for lw in self.model.layers):
            from .redundancy import RedundancyExpertManager

            self.redundancy = RedundancyExpertManager(self.model)

    def has_work(self) -> bool:
        return True  # the agreement inside step() decides; every rank must keep calling step()

    def _agree(self, n_prefill_tokens: int, n_decode: int):
        mine = torch.tensor([n_prefill_tokens, n_decode, len(self.ctx.requests)], dtype=torch.int64)
        if self.ps.world_size == 1 or self.ps.cpu_group is None:
            return mine.view(1, 3)
        allv = torch.empty(self.ps.world_size * 3, dtype=torch.int64)
        t0 = time.perf_counter()
        dist.all_gather_into_tensor(allv, mine, group=self.ps.cpu_group)
        self.stats["agree_s"] = self.stats.get("agree_s", 0.0) + (time.perf_counter() - t0)
        return allv.view(self.ps.world_size, 3)

    def _hold_input(self, is_prefill: bool) -> ModelInput:
        rm, mm = self.model.req_manager, self.model.mem_manager
        one = torch.ones(1, dtype=torch.int32)
        kw = dict(batch_size=1, total_token_num=1, max_kv_len=1, is_prefill=is_prefill,
                  b_req_idx=torch.tensor([rm.HOLD_REQUEST_ID], dtype=torch.int32), b_seq_len=one,
                  mem_indexes=torch.tensor([mm.HOLD_TOKEN_MEMINDEX], dtype=torch.int32))
        if is_prefill:
            kw.update(input_ids=torch.zeros(1, dtype=torch.int64), b_ready_cache_len=torch.zeros(1, dtype=torch.int32),
                      b_q_len=one, max_q_len=1)
        return ModelInput(**kw)

    @torch.no_grad()
    def step(self) -> dict:
        """One lock-step pass.  A plain decode step is launched before the previous step's tokens have been read back
        (as in the single-replica backend): the host-side bookkeeping of step k and the vote for step k + 1 run while
        the GPU executes, so a replica's GPU does not sit idle between passes and, through the layer-wise token
        exchanges, hold up every other replica."""
        self._steps += 1
        self._tick_tree_merge()      # every call is a lock-step over all ranks: the tick is the same everywhere
        if self.redundancy is not None and self.redundancy.step():
            self.stats["redundancy_updates"] = self.stats.get("redundancy_updates", 0) + 1
        prefill, decode, finished = self._get_classed_reqs()
        local_kind = self.control.select(len(prefill), len(decode))
        defer = local_kind == "decode" and self._can_defer(decode)
        if self._pending is not None and not defer:
            # settle the step in flight first, so that the vote says what this replica will really run
            self._flush_pending()
            prefill, decode, fin2 = self._get_classed_reqs()
            finished += [r for r in fin2 if r not in finished]
            local_kind = self.control.select(len(prefill), len(decode))
            defer = local_kind == "decode" and self._can_defer(decode)
        votes = self._agree(sum(c for _, c in prefill) if local_kind == "prefill" else 0,
                            len(decode) if local_kind == "decode" else 0)
        any_prefill, any_decode = bool((votes[:, 0] > 0).any()), bool((votes[:, 1] > 0).any())
        n_tok, kind = 0, "idle"
        if any_prefill:
            kind = "prefill"
            # every rank saw the same votes: the largest prompt chunk of this step bounds the expert exchange
            self.model.ep_prefill_tokens_bound = max(int(votes[:, 0].max()), 1)
            if local_kind == "prefill":
                n_tok = self._run_prefill(prefill)
            else:
                self._hold_pass(True)
                self.stats["hold_prefill"] += 1
        elif any_decode:
            kind = "decode"
            self._before_decode_round(int(votes[:, 1].max()))
            if local_kind == "decode":
                n_tok = self._run_decode(decode, defer=defer)
            else:
                self._hold_pass(False)
                self.stats["hold_decode"] += 1
        else:
            if self._pending is not None:
                self._flush_pending()
            else:
                time.sleep(self.idle_sleep_s)
        for req in list(self.ctx.requests.values()):
            if req.finish_status.is_finished() and req not in finished:
                finished.append(req)
        finished = [r for r in finished if not r.retire_hold]
        for req in finished:
            self.ctx.remove_req(req)
        # requests whose last token is still in flight are in the table, so the (shared) votes cover them:
        # every rank leaves drain() on the same step
        return {"kind": kind, "finished": finished, "tokens": n_tok, "world_busy": bool((votes[:, 2] > 0).any())}

    def _hold_pass(self, is_prefill: bool):
        """What an idle replica runs while the others work: the same sequence of model passes (every MoE layer of
        every pass is a collective), over the hold request."""
        self.model.forward(self._hold_input(is_prefill))

    def _before_decode_round(self, max_decode_reqs: int):
        """Hook: every replica knows the largest decode batch of the round."""

    def drain(self):
        """Keep stepping (holding) until no rank has a live request: a rank that finished early must stay in the
        exchanges of the others.  Every rank sees the same votes, so all of them leave on the same step."""
        while self.step()["world_busy"]:
            pass
