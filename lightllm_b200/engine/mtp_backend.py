"""Speculative decoding with multi-token-prediction draft modules.

Every decode step verifies the `k` draft tokens of each request in ONE pass of the target model: the inputs
of a request are [last output token, d_1 .. d_k] on top of its cached context (a prefill-shaped pass with k + 1
query tokens), the target's token at every position is sampled, and the longest prefix of drafts that equals
the target's own tokens is accepted.  The emitted tokens are always the target's samples, so the output
distribution is the target's; a request with penalties accepts no drafts (its logits depend on the emitted
tokens).  KV written for rejected positions is rolled back.  Then the draft module runs over the accepted
positions (target hidden state of position i + token i+1 -> proposal for token i+2); with k > 1 it is applied
recurrently on its own hidden state, writing its KV to scratch slots that are released after the step.

Reference: mode_backend/chunked_prefill/impl.py:244-446 (decode_mtp, vanilla / eagle draft loops),
common/basemodel/triton_kernel/mtp_utils.py (verify, accepted-token scatter).
"""
from __future__ import annotations

import time
from typing import List

import numpy as np
import torch

from .. import ops
from ..common.infer_state import ModelInput
from .backend import ModelBackend
from .dp_backend import DPBackend
from .infer_batch import InferReq


class MTPBackend(ModelBackend):
    def __init__(self, model, args=None, draft_models=None, mtp_step: int = 1, **kw):
        super().__init__(model, args, **kw)
        assert draft_models, "MTPBackend needs at least one draft module"
        self.drafts = draft_models
        self.k = int(mtp_step)
        self.stats.update({"mtp_steps": 0, "mtp_accepted": 0, "mtp_proposed": 0})

    # ------------------------------------------------------------------ helpers
    def _mi(self, reqs, ready, q_lens, slots, ids, **kw) -> ModelInput:
        ready = np.asarray(ready, dtype=np.int32)
        q_lens = np.asarray(q_lens, dtype=np.int32)
        return ModelInput(batch_size=len(reqs), total_token_num=int((ready + q_lens).sum()),
                          max_kv_len=int((ready + q_lens).max()), is_prefill=True,
                          b_req_idx=torch.tensor([r.req_idx for r in reqs], dtype=torch.int32),
                          b_seq_len=torch.from_numpy(ready + q_lens), mem_indexes=slots,
                          input_ids=torch.from_numpy(np.asarray(ids, dtype=np.int64)),
                          b_ready_cache_len=torch.from_numpy(ready), b_q_len=torch.from_numpy(q_lens),
                          max_q_len=int(q_lens.max()), **kw)

    def _propose(self, reqs: List[InferReq], ready, q_lens, slots, next_ids, hidden):
        """Draft pass over positions whose target hidden states are `hidden`; `next_ids[i]` is the token that
        follows position i.  Stores k proposals in r.extra["drafts"] for the requests in `reqs`."""
        d = self.drafts[0]
        out = d.forward(self._mi(reqs, ready, q_lens, slots, next_ids, draft_input_hidden=hidden, return_hidden=True))
        tok, _ = ops.sample(out.logits)          # greedy proposals (rows = last position of every request)
        proposals = [tok]
        if self.k > 1:
            last_rows = torch.from_numpy(np.cumsum(q_lens) - 1).to(self.device)
            h = out.hidden.index_select(0, last_rows)
            B = len(reqs)
            pos = np.asarray(ready, dtype=np.int32) + np.asarray(q_lens, dtype=np.int32)  # first scratch position
            scratch = self.ctx.alloc_slots(B * (self.k - 1)).view(B, self.k - 1)
            for j in range(1, self.k):
                mod = self.drafts[min(j, len(self.drafts) - 1)]
                mi = self._mi(reqs, pos + j - 1, np.ones(B, dtype=np.int32), scratch[:, j - 1].contiguous(),
                              proposals[-1].cpu().numpy(), draft_input_hidden=h, return_hidden=True)
                o = mod.forward(mi)
                t, _ = ops.sample(o.logits)
                proposals.append(t)
                h = o.hidden
            self.model.mem_manager.free(scratch.reshape(-1))
        props = torch.stack(proposals, dim=1).cpu().numpy()     # [B, k]
        for i, r in enumerate(reqs):
            r.extra["drafts"] = props[i].tolist()

    def _propose_nothing(self):
        """Hook for lock-step data parallelism: a step that has nothing to propose for (plain backend: no pass)."""

    # ------------------------------------------------------------------ prefill
    def _run_prefill(self, items) -> int:
        reqs = [r for r, _ in items]
        chunks = np.array([c for _, c in items], dtype=np.int32)
        ready = np.array([r.cur_kv_len for r in reqs], dtype=np.int32)
        total = int(chunks.sum())
        ids = np.concatenate([r.get_chunked_input_token_ids(int(c)) for r, c in items])
        slots = self.ctx.alloc_slots(total)
        slots_np, off = slots.numpy(), 0
        for r, c in items:
            r.slots = np.concatenate([r.slots[: r.cur_kv_len], slots_np[off:off + c]])
            off += int(c)
        out = self.model.forward(self._mi(reqs, ready, chunks, slots, ids, return_hidden=True))
        has_out = np.array([r.cur_kv_len + int(c) >= r.total_len() for r, c in items], dtype=bool)
        for r, c in items:
            r.cur_kv_len += int(c)
        if has_out.any():
            self._sample_and_post(reqs, out.logits, has_out, is_prefill=True)
        elif self.is_master_in_dp:
            for r in reqs:
                r.shm_req.shm_cur_kv_len = r.cur_kv_len
        # draft module over the same positions: token i+1 with the target's hidden state of position i
        nxt = np.empty(total, dtype=np.int64)
        off = 0
        for r, c in items:
            c = int(c)
            start = r.cur_kv_len - c
            nxt[off:off + c] = r.shm_req.shm_prompt_ids.arr[start + 1:start + c + 1]  # the sampled token is in place
            off += c
        self._propose(reqs, ready, chunks, slots, nxt, out.hidden)
        self.stats["prefill_steps"] += 1
        self.stats["prefill_tokens"] += total
        return int(has_out.sum())

    # ------------------------------------------------------------------ decode = verify + propose
    def _run_decode(self, reqs: List[InferReq], defer: bool = False) -> int:
        k, B = self.k, len(reqs)
        q = k + 1
        base = np.array([r.cur_kv_len for r in reqs], dtype=np.int32)
        ids = np.empty(B * q, dtype=np.int64)
        for i, r in enumerate(reqs):
            drafts = r.extra.get("drafts") or [0] * k
            ids[i * q] = r.get_last_gen_token()
            ids[i * q + 1:(i + 1) * q] = drafts[:k]
        slots = self.ctx.alloc_slots(B * q)
        slots_np = slots.numpy().reshape(B, q)
        for i, r in enumerate(reqs):
            r.slots = np.concatenate([r.slots[: r.cur_kv_len], slots_np[i]])
        rollback = getattr(self.model, "needs_state_rollback", False)   # models with recurrent per-request state
        out = self.model.forward(self._mi(reqs, base, np.full(B, q, dtype=np.int32), slots, ids,
                                          return_all_logits=True, return_hidden=True, verify_pass=rollback))
        logits = out.logits                                            # [B * q, V]
        first_rows = torch.arange(0, B * q, q, device=logits.device)
        if any(r.sampling.has_penalty for r in reqs):
            l0 = logits.index_select(0, first_rows)
            self._apply_penalties(reqs, l0)
            logits.index_copy_(0, first_rows, l0)
        rep = lambda xs, dt: torch.tensor(np.repeat(np.asarray(xs), q), dtype=dt).to(self.device)  # noqa: E731
        if all(r.sampling.top_k == 1 for r in reqs):
            tok, lps = ops.sample(logits)
        else:
            steps = np.concatenate([np.arange(r.cur_output_len, r.cur_output_len + q) for r in reqs])
            tok, lps = ops.sample(logits, rep([r.sampling.temperature for r in reqs], torch.float32),
                                  rep([r.sampling.top_p for r in reqs], torch.float32),
                                  rep([r.sampling.top_k for r in reqs], torch.int32),
                                  rep([r.seed for r in reqs], torch.int64),
                                  torch.tensor(steps, dtype=torch.int64).to(self.device))
        tok_np, lps_np = tok.cpu().numpy().reshape(B, q), lps.cpu().numpy().reshape(B, q)
        now = time.time()
        emitted = np.zeros(B, dtype=np.int32)
        for i, r in enumerate(reqs):
            drafts = ids[i * q + 1:(i + 1) * q]
            a = 0
            if not r.sampling.has_penalty:
                while a < k and int(drafts[a]) == int(tok_np[i, a]):
                    a += 1
            n_emit = 0
            for j in range(a + 1):
                r.append_token(int(tok_np[i, j]), float(lps_np[i, j]))
                n_emit += 1
                r.update_finish_status(self.eos_ids, self.args.max_req_total_len)
                if self.extra_post_req_handle_func is not None:
                    self.extra_post_req_handle_func(r, int(tok_np[i, j]), float(lps_np[i, j]))
                if r.finish_status.is_finished():
                    break
            emitted[i] = n_emit
            # KV of the inputs at positions base .. base + n_emit - 1 stays; the rest is rolled back
            keep = int(base[i]) + n_emit
            self.model.mem_manager.free(r.slots[keep:])
            r.slots = r.slots[:keep]
            r.cur_kv_len = keep
            r.shm_req.mtp_accepted_token_num += n_emit - 1
            self.stats["mtp_accepted"] += n_emit - 1
            self.stats["mtp_proposed"] += k
            if self.is_master_in_dp:
                if r.cur_output_len == n_emit:
                    r.shm_req.first_token_time = now
                r.publish()
            if self.on_token is not None:
                for j in range(n_emit):
                    self.on_token(r, int(tok_np[i, j]), float(lps_np[i, j]))
        if rollback:
            self.model.commit_verify(emitted)
        # next proposals from the accepted positions (requests that just finished need none)
        live = [i for i, r in enumerate(reqs) if not r.finish_status.is_finished()]
        if not live:
            self._propose_nothing()
        if live:
            rows = np.concatenate([np.arange(i * q, i * q + emitted[i]) for i in live])
            rows_t = torch.from_numpy(rows).to(self.device)
            lr = [reqs[i] for i in live]
            nxt = np.concatenate([tok_np[i, :emitted[i]] for i in live])
            d_slots = torch.from_numpy(np.concatenate([slots_np[i, :emitted[i]] for i in live]).astype(np.int32))
            self._propose(lr, base[live], emitted[live], d_slots, nxt, out.hidden.index_select(0, rows_t))
        self.stats["decode_steps"] += 1
        self.stats["mtp_steps"] += 1
        self.stats["decode_tokens"] += int(emitted.sum())
        return int(emitted.sum())


class DPMTPBackend(DPBackend, MTPBackend):
    """Speculative decoding under lock-step data parallelism (`--dp` > 1 with `--mtp_mode`): every replica runs the
    same sequence of model passes in a round (target pass, then `mtp_step` draft passes), whatever it has to do
    itself, because every MoE layer of every pass is an exchange among all replicas: an idle replica, or one whose
    requests all just finished, runs the passes over the hold request.  A decode round's target pass is the
    prompt-shaped verification pass, so the bound of the expert exchange is (largest decode batch) x (mtp_step + 1).
    Reference: lightllm/server/router/model_infer/mode_backend/dp_backend/impl.py (prefill_mtp / decode_mtp and
    their padded variants)."""

    def _hold_pass(self, is_prefill: bool):
        mi = self._hold_input(True)           # verification passes are prompt-shaped too
        mi.return_hidden = True
        out = self.model.forward(mi)
        self._hold_drafts(out.hidden)

    def _hold_drafts(self, hidden):
        h = hidden[-1:].contiguous() if hidden is not None else None
        for j in range(self.k):
            mod = self.drafts[min(j, len(self.drafts) - 1)]
            mi = self._hold_input(True)
            mi.draft_input_hidden, mi.return_hidden = h, True
            h = mod.forward(mi).hidden

    def _propose_nothing(self):
        self._hold_drafts(torch.zeros((1, self.model.hidden), dtype=self.model.dtype, device=self.device))

    def _before_decode_round(self, max_decode_reqs: int):
        self.model.ep_prefill_tokens_bound = max(1, max_decode_reqs * (self.k + 1))
