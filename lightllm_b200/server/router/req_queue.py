"""Admission queues of the router: the Past-Future scheduler and its variants.

A waiting request is admitted when the *simulated peak* KV demand of (running + candidate)
requests stays under the pool size.  Each request contributes a pair (a, b): a = tokens it
holds, b = tokens it is still expected to produce.  Sorting by b descending and scanning,
the peak demand is  max_i ( b_i * (i+1) + sum_{j<=i} a_j ): when request i finishes, the i+1
longest-living requests have each grown by b_i.  FCFS: the scan stops at the first request
that does not fit.

Reference: lightllm/server/router/req_queue/chunked_prefill/impl.py:24-93 (ChunkedPrefillQueue),
impl_for_pd.py (PD variant), beam_impl.py (shared-prefix groups), dp_base_queue.py + dp_balancer/.
"""
from __future__ import annotations

import random
from typing import List, Optional, Tuple

import numpy as np

from ..core.objs.req import Req


class RouterStatics:
    """Moving average of finished output lengths; the smoothing factor decays 0.5 -> 0.04 so early
    samples move the estimate quickly (reference: lightllm/server/router/stats.py)."""

    def __init__(self, init_len: int = 2048, floor: int = 64):
        self.ema_req_out_len = init_len
        self.floor = floor
        self.alpha = 0.5
        self.min_alpha = 0.04

    def update(self, req_out_len: int):
        self.ema_req_out_len = int(self.ema_req_out_len * (1 - self.alpha) + req_out_len * self.alpha)
        self.ema_req_out_len = max(self.floor, self.ema_req_out_len)
        self.alpha = max(self.min_alpha, self.alpha * 0.9)


class Batch:
    def __init__(self, batch_id: int, reqs: List[Req], dp_size_in_node: int = 1):
        self.batch_id = batch_id
        self.reqs = list(reqs)
        self.id_to_reqs = {r.request_id: r for r in reqs}
        self.dp_size_in_node = dp_size_in_node

    def input_tokens(self) -> int:
        return sum(r.input_len for r in self.reqs)

    def get_req_list_for_dp(self, dp_index: int) -> List[Req]:
        if self.dp_size_in_node == 1:
            return self.reqs
        return [r for r in self.reqs if r.sample_params.suggested_dp_index == dp_index]

    def filter_out_finished_req(self, shm_req_manager=None) -> List[Req]:
        """Drops requests the model ranks have released; returns them."""
        done = [r for r in self.reqs if r.shm_infer_released]
        if done:
            self.reqs = [r for r in self.reqs if not r.shm_infer_released]
            self.id_to_reqs = {r.request_id: r for r in self.reqs}
            if shm_req_manager is not None:
                for r in done:
                    shm_req_manager.put_back_req_obj(r)
        return done

    def pop_req(self, req_id):
        r = self.id_to_reqs.pop(req_id)
        self.reqs.remove(r)
        return r

    def is_clear(self) -> bool:
        return len(self.reqs) == 0

    def merge(self, other: Optional["Batch"]):
        if other is None:
            return
        for r in other.reqs:
            self.reqs.append(r)
            self.id_to_reqs[r.request_id] = r

    def __len__(self):
        return len(self.reqs)


class BaseQueue:
    def __init__(self, max_total_tokens: int, batch_max_tokens: int, running_max_req_size: int,
                 router_token_ratio: float = 0.85, dp_index: int = 0, dp_size_in_node: int = 1,
                 statics: Optional[RouterStatics] = None, token_load=None):
        self.max_total_tokens = max_total_tokens
        self.batch_max_tokens = batch_max_tokens
        self.running_max_req_size = running_max_req_size
        self.router_token_ratio = router_token_ratio
        self.dp_index = dp_index
        self.dp_size_in_node = dp_size_in_node
        self.waiting_req_list: List[Req] = []
        self.statics = statics or RouterStatics()
        self.token_load = token_load
        self.cur_token_usage_ratio = 0.0  # set by the router from the ranks' published free-token counters

    def append(self, req: Req):
        req.sample_params.suggested_dp_index = self.dp_index
        self.waiting_req_list.append(req)

    def extend(self, reqs):
        for r in reqs:
            self.append(r)

    def get_wait_req_num(self) -> int:
        return len(self.waiting_req_list)

    def is_busy(self) -> bool:
        return self.cur_token_usage_ratio >= self.router_token_ratio

    def free_aborted_req_cache_tokens(self):
        pass

    def pop_aborted(self) -> List[Req]:
        """Waiting requests whose client went away are released by the router itself."""
        gone = [r for r in self.waiting_req_list if r.is_aborted]
        if gone:
            self.waiting_req_list = [r for r in self.waiting_req_list if not r.is_aborted]
        return gone


class PeakEstimate:
    """Past-Future estimate of the largest KV footprint a set of requests will reach.

    Every request contributes (held, growth): tokens it holds once its prompt is in, and tokens it is still expected
    to produce.  Requests finish in order of remaining growth; just before the request with the i-th largest
    growth g_i finishes, the i requests that outlive the others have each grown by g_i, on top of what those i
    hold now: peak = max_i (i * g_i + sum of `held` over the i largest growths).
    Reference: lightllm/server/router/req_queue/chunked_prefill/impl.py:22-51."""

    def __init__(self, pairs=()):
        self.pairs: List[Tuple[int, int]] = list(pairs)

    def copy(self) -> "PeakEstimate":
        return PeakEstimate(self.pairs)

    def add(self, held: int, growth: int):
        self.pairs.append((int(held), int(growth)))

    def __len__(self):
        return len(self.pairs)

    def peak(self) -> int:
        if not self.pairs:
            return 0
        arr = np.array(sorted(self.pairs, key=lambda p: -p[1]), dtype=np.int64)
        alive = np.arange(1, arr.shape[0] + 1, dtype=np.int64)
        return int((arr[:, 1] * alive + np.cumsum(arr[:, 0])).max())

    def held(self) -> int:
        return int(sum(p[0] for p in self.pairs))


class ChunkedPrefillQueue(BaseQueue):
    PREFILL_PASSES_OF_SLACK = 2   # a new batch may queue up to this many forward passes of prompt tokens

    def _tuple_of(self, req: Req, is_busy: bool):
        return req.get_tuple_tokens(is_busy, self.statics.ema_req_out_len)

    def _estimate_of(self, current_batch: Optional[Batch], is_busy: bool) -> PeakEstimate:
        est = PeakEstimate()
        if current_batch is not None:
            for r in current_batch.get_req_list_for_dp(self.dp_index):
                est.add(*self._tuple_of(r, is_busy))
        return est

    def _admit(self, est: PeakEstimate, req: Req, is_busy: bool, prefill_tokens: int):
        """Adds `req` to the estimate; returns (fits, prompt tokens the next passes would then have to run)."""
        est.add(*self._tuple_of(req, is_busy))
        prefill_tokens += req.get_first_router_need_tokens()
        fits = (est.peak() < self.max_total_tokens and len(est) <= self.running_max_req_size
                and prefill_tokens <= self.PREFILL_PASSES_OF_SLACK * self.batch_max_tokens)
        return fits, prefill_tokens

    def _running_need(self, current_batch: Optional[Batch]) -> int:
        """Tokens the next pass already owes to the running requests of this replica (one per decoding request,
        the next chunk of a prompt still being prefilled); new prompts are budgeted on top of it
        (reference: chunked_prefill/impl.py:67-69)."""
        if current_batch is None:
            return 0
        return sum(r.get_decode_need_tokens() for r in current_batch.get_req_list_for_dp(self.dp_index))

    def take(self, group_req_ids: List[int], next_batch_id: int = 0) -> Optional[Batch]:
        """Admits exactly the requests of these groups, in the given order, without consulting the estimate
        (multi-node tensor parallelism: the master node's router has decided for everybody)."""
        if not group_req_ids:
            return None
        order = {g: i for i, g in enumerate(group_req_ids)}
        chosen = sorted((r for r in self.waiting_req_list if r.group_req_id in order),
                        key=lambda r: (order[r.group_req_id], r.request_id))
        taken = {id(r) for r in chosen}
        self.waiting_req_list = [r for r in self.waiting_req_list if id(r) not in taken]
        return Batch(next_batch_id, chosen, self.dp_size_in_node) if chosen else None

    def generate_new_batch(self, current_batch: Optional[Batch], next_batch_id: int = 0,
                           allowed_groups=None) -> Optional[Batch]:
        """`allowed_groups`: only requests of these group ids may be admitted (the scan stops at the first waiting
        request outside it, keeping the order first come, first served)."""
        if not self.waiting_req_list:
            return None
        running = len(current_batch.get_req_list_for_dp(self.dp_index)) if current_batch is not None else 0
        if running >= self.running_max_req_size:
            return None
        is_busy = self.is_busy()
        est = self._estimate_of(current_batch, is_busy)
        prefill_tokens = self._running_need(current_batch)
        can_run = []
        for req in self.waiting_req_list:
            if req.is_aborted:  # released by the router, never scheduled
                continue
            if allowed_groups is not None and req.group_req_id not in allowed_groups:
                break
            ok, prefill_tokens = self._admit(est, req, is_busy, prefill_tokens)
            if not ok:
                break
            can_run.append(req)
        if not can_run:
            return None
        taken = {id(r) for r in can_run}
        self.waiting_req_list = [r for r in self.waiting_req_list if id(r) not in taken]
        return Batch(next_batch_id, can_run, self.dp_size_in_node)

    def calcu_batch_token_load(self, current_batch: Optional[Batch]):
        """(estimated peak ratio, current used ratio) for /token_load."""
        est = self._estimate_of(current_batch, self.is_busy())
        if not len(est):
            return 0.0, 0.0
        return est.peak() / self.max_total_tokens, est.held() / self.max_total_tokens


class PDQueue(ChunkedPrefillQueue):
    """Prefill/decode-disaggregated nodes: a request not yet decoding is counted at its full length."""

    def _tuple_of(self, req: Req, is_busy: bool):
        if req.shm_cur_output_len == 0:
            return req.input_len + 1, req.sample_params.max_new_tokens + 16
        return super()._tuple_of(req, is_busy)


class ChunkedBeamContinuesBatchQueue(ChunkedPrefillQueue):
    """diverse_mode: the n samples of a group share their prompt KV; admit or reject the whole group."""

    def generate_new_batch(self, current_batch, next_batch_id: int = 0):
        if not self.waiting_req_list:
            return None
        is_busy = self.is_busy()
        est = self._estimate_of(current_batch, is_busy)
        groups, order = {}, []
        for r in self.waiting_req_list:
            if r.group_req_id not in groups:
                groups[r.group_req_id] = []
                order.append(r.group_req_id)
            groups[r.group_req_id].append(r)
        can_run, prefill_tokens = [], self._running_need(current_batch)
        for gid in order:
            trial = est.copy()
            ok_all, after = True, prefill_tokens
            for i, r in enumerate(groups[gid]):
                # the group's prompt is prefilled once: only its first member adds prompt tokens to the passes
                ok, t = self._admit(trial, r, is_busy, prefill_tokens if i == 0 else
                                    after - r.get_first_router_need_tokens())
                if i == 0:
                    after = t
                if not ok:
                    ok_all = False
                    break
            if not ok_all:
                break
            est, prefill_tokens = trial, after
            can_run.extend(groups[gid])
        if not can_run:
            return None
        taken = {id(r) for r in can_run}
        self.waiting_req_list = [r for r in self.waiting_req_list if id(r) not in taken]
        return Batch(next_batch_id, can_run, self.dp_size_in_node)


# ---- data-parallel attention: one inner queue per replica + a balancer ----
class DpBalancer:
    def __init__(self, dp_size_in_node: int, inner_queues: List[BaseQueue]):
        self.dp_size_in_node = dp_size_in_node
        self.inner_queues = inner_queues

    def assign_reqs_to_dp(self, current_batch: Optional[Batch], reqs: List[Req]):
        raise NotImplementedError


class RoundRobinDpBalancer(DpBalancer):
    def __init__(self, *a):
        super().__init__(*a)
        self._next = 0

    def assign_reqs_to_dp(self, current_batch, reqs):
        for r in reqs:
            idx = r.sample_params.suggested_dp_index
            if not (0 <= idx < self.dp_size_in_node):
                idx = self._next
                self._next = (self._next + 1) % self.dp_size_in_node
            self.inner_queues[idx].append(r)


class DpBsBalancer(DpBalancer):
    """Least (running + waiting) requests first, random tie-break."""

    def assign_reqs_to_dp(self, current_batch, reqs):
        counts = [q.get_wait_req_num() for q in self.inner_queues]
        if current_batch is not None:
            for r in current_batch.reqs:
                i = r.sample_params.suggested_dp_index
                if 0 <= i < self.dp_size_in_node:
                    counts[i] += 1
        for r in reqs:
            idx = r.sample_params.suggested_dp_index
            if not (0 <= idx < self.dp_size_in_node):
                low = min(counts)
                idx = random.choice([i for i, c in enumerate(counts) if c == low])
            counts[idx] += 1
            self.inner_queues[idx].append(r)


class DpQueue:
    def __init__(self, inner_cls, dp_size_in_node: int, balancer: str = "bs_balancer", **kw):
        self.dp_size_in_node = dp_size_in_node
        self.inner_queues = [inner_cls(dp_index=i, dp_size_in_node=dp_size_in_node, **kw)
                             for i in range(dp_size_in_node)]
        cls = RoundRobinDpBalancer if balancer == "round_robin" else DpBsBalancer
        self.balancer = cls(dp_size_in_node, self.inner_queues)
        self._pending: List[Req] = []

    def append(self, req):
        self._pending.append(req)

    def extend(self, reqs):
        self._pending.extend(reqs)

    def get_wait_req_num(self):
        return sum(q.get_wait_req_num() for q in self.inner_queues) + len(self._pending)

    def set_usage(self, ratios):
        for q, r in zip(self.inner_queues, ratios):
            q.cur_token_usage_ratio = r

    def pop_aborted(self):
        out = [r for r in self._pending if r.is_aborted]
        self._pending = [r for r in self._pending if not r.is_aborted]
        for q in self.inner_queues:
            out += q.pop_aborted()
        return out

    def generate_new_batch(self, current_batch, next_batch_id: int = 0):
        if self._pending:
            self.balancer.assign_reqs_to_dp(current_batch, self._pending)
            self._pending = []
        merged = None
        for q in self.inner_queues:
            b = q.generate_new_batch(current_batch, next_batch_id)
            if b is not None:
                if merged is None:
                    merged = b
                else:
                    merged.merge(b)
        return merged

    def calcu_batch_token_load(self, current_batch):
        return [q.calcu_batch_token_load(current_batch) for q in self.inner_queues]


def build_req_queue(args, max_total_tokens: int, dp_size_in_node: int = 1, statics=None):
    """Queue class from the launch flags (reference: lightllm/server/router/req_queue/__init__.py:27-33)."""
    if getattr(args, "run_mode", "normal") in ("prefill", "decode"):
        cls = PDQueue
    elif getattr(args, "diverse_mode", False):
        cls = ChunkedBeamContinuesBatchQueue
    else:
        cls = ChunkedPrefillQueue
    kw = dict(max_total_tokens=max_total_tokens, batch_max_tokens=args.batch_max_tokens,
              running_max_req_size=args.running_max_req_size, router_token_ratio=args.router_token_ratio,
              statics=statics)
    if dp_size_in_node == 1:
        return cls(**kw)
    return DpQueue(cls, dp_size_in_node, getattr(args, "dp_balancer", "bs_balancer"), **kw)
