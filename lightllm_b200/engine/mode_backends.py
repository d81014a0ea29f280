"""Backend variants selected by launch flags.  Each one is `ModelBackend` plus hooks:
logit masks before sampling (`prefill_mask_func` / `decode_mask_func`) and a per-token post
handler (`extra_post_req_handle_func`).

Reference: lightllm/server/router/model_infer/mode_backend/* (TokenHealingBackend,
OutlinesConstraintBackend, XgrammarBackend, FirstTokenConstraintBackend, RewardModelBackend,
DiversehBackend) and model_rpc.py:72-99 (selection).
"""
from __future__ import annotations

import os
import time
from typing import List

import numpy as np
import torch

from .backend import ModelBackend
from .infer_batch import InferReq


class FirstTokenConstraintBackend(ModelBackend):
    """Only the ids in env FIRST_ALLOWED_TOKENS (comma separated) may be generated first."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        allowed = [int(t) for t in os.environ.get("FIRST_ALLOWED_TOKENS", "").split(",") if t.strip()]
        assert allowed, "set FIRST_ALLOWED_TOKENS=id,id,..."
        self._allowed = torch.tensor(allowed, dtype=torch.long)
        self.prefill_mask_func = self._mask

    def _mask(self, reqs: List[InferReq], logits: torch.Tensor):
        keep = self._allowed.to(logits.device)
        m = torch.full_like(logits, float("-inf"))
        m[:, keep] = 0.0
        for i, r in enumerate(reqs):
            if r.cur_output_len == 0:
                logits[i] += m[i]


class TokenHealingBackend(ModelBackend):
    """The last prompt tokens were cut off (TokenHealingReq); generation is constrained to tokens whose
    text continues the removed text until it is covered again."""

    def __init__(self, *a, tokenizer=None, **kw):
        super().__init__(*a, **kw)
        self.tokenizer = tokenizer
        self._vocab_strs = None
        self.prefill_mask_func = self._mask
        self.decode_mask_func = self._mask
        self.extra_post_req_handle_func = self._after_token

    def _vocab(self):
        if self._vocab_strs is None:
            V = self.model.vocab
            toks = self.tokenizer.convert_ids_to_tokens(list(range(V))) if self.tokenizer is not None else None
            self._vocab_strs = [t if isinstance(t, str) else "" for t in (toks or [""] * V)]
        return self._vocab_strs

    def _state(self, r: InferReq):
        st = r.extra.get("heal")
        if st is None:
            ids = r.shm_req.prefix_token_ids.to_list()
            text = "".join(self.tokenizer.convert_ids_to_tokens(ids)) if (ids and self.tokenizer is not None) else ""
            st = r.extra["heal"] = {"remaining": text}
        return st

    def _mask(self, reqs, logits):
        for i, r in enumerate(reqs):
            rem = self._state(r)["remaining"]
            if not rem:
                continue
            ok = [j for j, s in enumerate(self._vocab()) if s and (s.startswith(rem) or rem.startswith(s))]
            if ok:
                m = torch.full((logits.shape[1],), float("-inf"), device=logits.device)
                m[torch.tensor(ok, device=logits.device)] = 0.0
                logits[i] += m

    def _after_token(self, r: InferReq, tok: int, lp: float):
        st = self._state(r)
        if st["remaining"]:
            s = self._vocab()[tok]
            st["remaining"] = st["remaining"][len(s):] if st["remaining"].startswith(s) else ""


class XgrammarBackend(ModelBackend):
    """EBNF / JSON-schema constrained decoding through xgrammar token bitmasks."""

    def __init__(self, *a, tokenizer=None, tokenizer_info=None, **kw):
        super().__init__(*a, **kw)
        import xgrammar as xgr

        self.xgr = xgr
        info = tokenizer_info if tokenizer_info is not None else \
            xgr.TokenizerInfo.from_huggingface(tokenizer, vocab_size=self.model.vocab)
        self.compiler = xgr.GrammarCompiler(info, max_threads=8)
        self.prefill_mask_func = self._mask
        self.decode_mask_func = self._mask
        self.extra_post_req_handle_func = self._after_token

    def _matcher(self, r: InferReq):
        m = r.extra.get("xgr", False)
        if m is False:
            sp = r.sampling
            if sp.guided_grammar == "json":
                cg = self.compiler.compile_builtin_json_grammar()
            elif sp.guided_grammar:
                cg = self.compiler.compile_grammar(sp.guided_grammar)
            elif sp.guided_json:
                cg = self.compiler.compile_json_schema(sp.guided_json)
            elif sp.regular_constraint:   # regular expressions run on the same matcher (no outlines needed)
                cg = self.compiler.compile_regex(sp.regular_constraint)
            else:
                cg = None
            m = r.extra["xgr"] = self.xgr.GrammarMatcher(cg) if cg is not None else None
        return m

    def _mask(self, reqs, logits):
        rows = [(i, self._matcher(r)) for i, r in enumerate(reqs)]
        rows = [(i, m) for i, m in rows if m is not None]
        if not rows:
            return
        bitmask = self.xgr.allocate_token_bitmask(len(rows), self.model.vocab)
        for j, (i, m) in enumerate(rows):
            m.fill_next_token_bitmask(bitmask, j)
        idx = torch.tensor([i for i, _ in rows], device=logits.device)
        sub = logits[idx]
        self.xgr.apply_token_bitmask_inplace(sub, bitmask.to(logits.device))
        logits[idx] = sub

    def _after_token(self, r: InferReq, tok: int, lp: float):
        m = self._matcher(r)
        if m is not None:
            if not m.accept_token(tok) or m.is_terminated():
                from ..server.core.objs.req import FinishStatus

                r.finish_status.set_status(FinishStatus.FINISHED_STOP)


class OutlinesConstraintBackend(ModelBackend):
    """Regex-constrained decoding with an outlines finite-state index (`outlines_core`: Vocabulary, Index, Guide):
    every request with `regular_constraint` walks its own guide; the tokens the current state allows are the only
    ones left in the logits, and the request stops when the guide is finished.  The index of a pattern is built
    once and shared.  Reference: mode_backend/continues_batch/outlines_constraint/impl.py."""

    def __init__(self, *a, tokenizer=None, vocabulary=None, **kw):
        super().__init__(*a, **kw)
        try:
            import outlines_core as oc
        except Exception as e:  # pragma: no cover
            raise RuntimeError("--output_constraint_mode outlines needs the `outlines_core` package; "
                               "use xgrammar instead") from e
        self.oc = oc
        self.eos = int(min(self.eos_ids)) if self.eos_ids else 0
        self.vocabulary = vocabulary if vocabulary is not None else self._vocabulary_of(tokenizer)
        self._indexes = {}
        self.prefill_mask_func = self._mask
        self.decode_mask_func = self._mask
        self.extra_post_req_handle_func = self._after_token

    def _vocabulary_of(self, tokenizer):
        V = self.model.vocab
        try:
            n = min(V, len(tokenizer))
        except TypeError:
            n = V
        toks = tokenizer.convert_ids_to_tokens(list(range(n)))
        table = {}
        for i, t in enumerate(toks):
            if i in self.eos_ids or not isinstance(t, str):
                continue
            try:
                text = tokenizer.convert_tokens_to_string([t])
            except Exception:
                text = t
            if text:
                table.setdefault(text, []).append(i)
        return self.oc.Vocabulary(self.eos, table)

    def _guide(self, r: InferReq):
        g = r.extra.get("guide", False)
        if g is False:
            pat = r.sampling.regular_constraint
            if pat:
                idx = self._indexes.get(pat)
                if idx is None:
                    idx = self._indexes[pat] = self.oc.Index(pat, self.vocabulary)
                g = self.oc.Guide(idx)
            else:
                g = None
            r.extra["guide"] = g
        return g

    def _mask(self, reqs, logits):
        for i, r in enumerate(reqs):
            g = self._guide(r)
            if g is None:
                continue
            allowed = torch.tensor(sorted(g.get_tokens()), dtype=torch.long, device=logits.device)
            m = torch.full((logits.shape[1],), float("-inf"), device=logits.device)
            m[allowed] = 0.0
            logits[i] += m

    def _after_token(self, r: InferReq, tok: int, lp: float):
        g = self._guide(r)
        if g is None:
            return
        from ..server.core.objs.req import FinishStatus

        if tok == self.eos or g.is_finished():
            r.finish_status.set_status(FinishStatus.FINISHED_STOP)
            return
        g.advance(tok)
        if g.is_finished():
            r.finish_status.set_status(FinishStatus.FINISHED_STOP)


class RewardModelBackend(ModelBackend):
    """Reward models: one prefill, the score head output is stored in `reward_score`; no decoding."""

    sharded_sampling = False   # reads a column of the dense matrix

    def _sample_and_post(self, reqs, logits, has_out, is_prefill):
        from ..server.core.objs.req import FinishStatus

        scores = logits[:, 0].float().cpu().numpy()
        for i, r in enumerate(reqs):
            if not has_out[i]:
                continue
            r.shm_req.reward_score = float(scores[i])
            r.append_token(0, 0.0)
            r.finish_status.set_status(FinishStatus.FINISHED_STOP)
            if self.is_master_in_dp:
                r.publish()


class DiverseBackend(ModelBackend):
    """n > 1 samples of one prompt: the first sub-request prefills, its KV goes to the radix tree
    right away, and its siblings match it instead of recomputing the prompt."""

    def add_reqs(self, shm_reqs):
        out = []
        by_group = {}
        for r in shm_reqs:
            by_group.setdefault(r.group_req_id, []).append(r)
        for group in by_group.values():
            out += super().add_reqs(group[:1])
            self._deferred = getattr(self, "_deferred", []) + group[1:]
        return out

    def step(self):
        res = super().step()
        deferred = getattr(self, "_deferred", [])
        if deferred and self.radix_cache is not None:
            ready, wait = [], []
            for r in deferred:
                master = self.ctx.requests.get(r.group_req_id)
                if master is None or master.cur_output_len > 0:
                    ready.append(r)
                else:
                    wait.append(r)
            for r in ready:
                master = self.ctx.requests.get(r.group_req_id)
                if master is not None:  # publish the prompt KV so that siblings hit it
                    n = r.input_len - 1
                    if n > 0:
                        self.radix_cache.insert(master.shm_req.shm_prompt_ids.arr[:n], master.slots[:n])
                        if master.shared_kv_node is not None:
                            self.radix_cache.dec_node_ref_counter(master.shared_kv_node)
                        node, m, _ = self.radix_cache.match_prefix(master.shm_req.shm_prompt_ids.arr[:n], True)
                        master.shared_kv_node, master.shared_len = node, m
                super().add_reqs([r])
            self._deferred = wait
        return res


def decode_replica_of(master_req_id: int, decode_dp: int) -> int:
    """The replica of a data-parallel decode node that serves a request: both sides compute it from the master's
    request id (ids advance in steps of 8), the prefill side to address the KV, the decode side to place the
    follow-up request."""
    return (int(master_req_id) // 8) % max(1, int(decode_dp))


class PDPrefillBackend(ModelBackend):
    """Prefill node of a disaggregated deployment: when a request's first token is sampled, its prompt KV is
    streamed to the paired decode rank (same tp rank) by a worker thread while the inference loop goes on with
    other requests.  The request stays in the table (slots referenced, first token not yet published) until the
    transfer has ended on every tensor-parallel rank; a failed transfer ends it with FINISHED_ERROR.
    Reference: mode_backend/pd/prefill_node_impl/prefill_impl.py:50-92 (its transfers run in a separate
    kv-move process)."""

    MAX_SETTLE = 64   # transfers whose outcome the ranks compare per step

    def __init__(self, *a, tp_rank: int = 0, page_tokens: int = 1024, cpu_group=None, tp_size: int = 1, **kw):
        super().__init__(*a, **kw)
        from .pd import KVSender

        self.tp_rank = tp_rank
        self.cpu_group, self.tp_size = cpu_group, tp_size
        self.sender = KVSender(self.model.mem_manager, page_tokens)
        self.extra_post_req_handle_func = self._ship
        self._sending = []      # [(InferReq, token, logprob)] in submission order (the same on every rank)
        self._outcome = {}      # req_id -> (ok, message) as seen by this rank's worker

    def _wants_ship(self, r: InferReq):
        params = r.shm_req.sample_params.pd_kv_trans_params.to_dict()
        return params if (params and r.cur_output_len == 1) else None

    def _ship(self, r: InferReq, tok: int, lp: float):
        params = self._wants_ship(r)
        if params is None:
            return
        r.retire_hold = True
        self._submit(r, params, tok, lp)

    def _submit(self, r: InferReq, params: dict, tok: int, lp: float):
        n = r.cur_kv_len
        ids = r.shm_req.shm_prompt_ids.arr[:n].tolist()
        self._sending.append(r)
        # rank (replica j, tensor-parallel rank t) of the decode node listens on its port base + j * (ranks per
        # replica) + t; P and D replicas have the same number of ranks
        d_dp, d_tp = int(params.get("decode_dp", 1) or 1), int(params.get("decode_tp", 1) or 1)
        per = max(1, d_tp // d_dp)
        port = params["peer_port"] + decode_replica_of(params["master_req_id"], d_dp) * per + self.tp_rank
        self.sender.submit((params["peer_ip"], port), params["master_req_id"], ids,
                           torch.from_numpy(np.ascontiguousarray(r.slots[:n])), (tok, lp), tag=r.req_id)

    def _settle_sends(self):
        """Ends the requests whose transfer is over.  With tensor parallelism every rank sends its own KV shard;
        a request is released on the step at which ALL ranks have an outcome for it (one small host all-reduce
        per step while transfers are pending), so the ranks' pools and schedules stay identical."""
        if not self._sending:
            return
        for tag, ok, msg in self.sender.poll_done():
            self._outcome[tag] = (ok, msg)
        head = self._sending[: self.MAX_SETTLE]
        state = torch.zeros(self.MAX_SETTLE, dtype=torch.int32)     # 0 pending, 1 sent, 2 failed
        for i, r in enumerate(head):
            o = self._outcome.get(r.req_id)
            if o is not None:
                state[i] = 1 if o[0] else 2
        if self.tp_size > 1 and self.cpu_group is not None:
            import torch.distributed as dist

            lo, hi = state.clone(), state.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=self.cpu_group)   # 0 while any rank is still sending
            dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self.cpu_group)   # 2 if any rank failed
            state = torch.where(lo == 0, lo, hi)
        keep = []
        for i, r in enumerate(head):
            st = int(state[i])
            if st == 0:
                keep.append(r)
                continue
            o = self._outcome.pop(r.req_id, None)
            if st == 2:
                from ..server.core.objs.req import FinishStatus

                print(f"[pd prefill] KV transfer of request {r.req_id} failed: {o[1] if o else 'on another rank'}",
                      flush=True)
                r.finish_status.set_status(FinishStatus.FINISHED_ERROR)
            r.retire_hold = False
            if self.is_master_in_dp:
                r.shm_req.first_token_time = time.time()
                r.publish()
        self._sending = keep + self._sending[self.MAX_SETTLE:]

    def has_work(self) -> bool:
        return super().has_work() or bool(self._sending)

    def step(self) -> dict:
        self._settle_sends()
        res = super().step()
        if res["kind"] == "idle" and self._sending:
            time.sleep(0.001)   # nothing to compute: wait for the worker without spinning
        return res


class PDDecodeBackend(ModelBackend):
    """Decode node: lands KV pages from prefill ranks between steps and publishes complete prompts to the
    prefix cache, so that the follow-up request (prompt + first token) starts decoding at once.
    `on_kv_done(group_req_id, ok)` is called on the master rank for each completed transfer.
    Reference: mode_backend/pd/decode_node_impl/decode_impl.py, up_status.py."""

    def __init__(self, *a, tp_rank: int = 0, host: str = "127.0.0.1", kv_port: int = 0, page_tokens: int = 1024,
                 page_num: int = 16, cpu_group=None, tp_size: int = 1, on_kv_done=None, **kw):
        super().__init__(*a, **kw)
        from .pd import KVReceiver

        assert self.radix_cache is not None, "a decode node needs the prefix cache (it is how transferred KV is found)"
        self.receiver = KVReceiver(self.model.mem_manager, host, kv_port + tp_rank if kv_port else 0, page_tokens, page_num)
        self.cpu_group, self.tp_size, self.on_kv_done = cpu_group, tp_size, on_kv_done

    MAX_KEYS = 64

    def _agree(self, keys):
        """Keys landed on every tp rank: one fixed-size all-gather on the host group."""
        import torch.distributed as dist

        mine = torch.full((self.MAX_KEYS,), -1, dtype=torch.int64)
        k = keys[: self.MAX_KEYS]
        mine[: len(k)] = torch.tensor(k, dtype=torch.int64)
        flat = torch.empty(self.tp_size * self.MAX_KEYS, dtype=torch.int64)   # gloo wants the output one-dimensional
        dist.all_gather_into_tensor(flat, mine, group=self.cpu_group)
        allk = flat.view(self.tp_size, self.MAX_KEYS)
        common = set(allk[0].tolist())
        for i in range(1, self.tp_size):
            common &= set(allk[i].tolist())
        common.discard(-1)
        return sorted(common)

    def has_work(self) -> bool:
        # with tp > 1 every rank must enter step() together: the agreement is a collective
        return super().has_work() or (self.tp_size == 1 and self.receiver.has_landed())

    def poll_kv(self):
        agree = self._agree if (self.tp_size > 1 and self.cpu_group is not None) else None
        for gid, ok, _first in self.receiver.drain(self.radix_cache, agree):
            if self.on_kv_done is not None and self.is_master_in_dp:
                self.on_kv_done(gid, ok)


def _pd_dp_classes():
    from .dp_backend import DPBackend

    class PDDPPrefillBackend(DPBackend, PDPrefillBackend):
        """Prefill node with data-parallel replicas (`--run_mode prefill --dp` > 1): the lock-step rounds of the
        data-parallel backend, KV shipped to the decode replica that will serve the request.  One rank per replica
        (the agreement among a replica's tensor-parallel ranks on settled transfers has no host group here).
        Reference: mode_backend/pd/prefill_node_impl/prefill_impl_for_dp.py."""

        def step(self) -> dict:
            self._settle_sends()
            return DPBackend.step(self)

    class PDDPDecodeBackend(DPBackend, PDDecodeBackend):
        """Decode node with data-parallel replicas: every rank lands the KV pages addressed to it between the
        lock-step rounds.  Reference: mode_backend/pd/decode_node_impl/decode_impl_for_dp.py."""

    return PDDPPrefillBackend, PDDPDecodeBackend


def pd_mtp_classes():
    """P/D node backends with speculative decoding (`--mtp_mode` on a prefill / decode node).  The KV pool carries
    the draft modules' layers, so the prefill node runs the draft pass over the prompt before it ships the pages
    (the hook only marks the request at sampling time, the transfer is submitted after the draft pass), and the
    decode node verifies and proposes as the plain speculative backend does.
    Reference: mode_backend/chunked_prefill/impl.py:244-446 run by the pd backends."""
    from .mtp_backend import MTPBackend

    class PDPrefillMTPBackend(PDPrefillBackend, MTPBackend):
        def __init__(self, *a, **kw):
            super().__init__(*a, **kw)
            self._ship_after_drafts = []
            self.extra_post_req_handle_func = self._mark_for_shipping

        def _mark_for_shipping(self, r: InferReq, tok: int, lp: float):
            params = self._wants_ship(r)
            if params is not None:
                r.retire_hold = True
                self._ship_after_drafts.append((r, params, tok, lp))

        def _run_prefill(self, items) -> int:
            n = MTPBackend._run_prefill(self, items)
            marked, self._ship_after_drafts = self._ship_after_drafts, []
            for r, params, tok, lp in marked:
                self._submit(r, params, tok, lp)
            return n

    class PDDecodeMTPBackend(PDDecodeBackend, MTPBackend):
        pass

    return PDPrefillMTPBackend, PDDecodeMTPBackend


def select_backend_class(args):
    if int(getattr(args, "dp", 1) or 1) > 1:
        from .dp_backend import DPBackend

        mode = getattr(args, "run_mode", "normal")
        if mode in ("prefill", "decode"):
            assert int(args.tp) == int(args.dp), "P/D nodes with --dp > 1 run one rank per replica (--dp equal to --tp)"
            return _pd_dp_classes()[0 if mode == "prefill" else 1]
        return DPBackend
    if getattr(args, "run_mode", "normal") == "prefill":
        return PDPrefillBackend
    if getattr(args, "run_mode", "normal") == "decode":
        return PDDecodeBackend
    if getattr(args, "use_reward_model", False):
        return RewardModelBackend
    if getattr(args, "token_healing_mode", False):
        return TokenHealingBackend
    mode = getattr(args, "output_constraint_mode", "none")
    if mode == "xgrammar":
        return XgrammarBackend
    if mode == "outlines":
        try:  # regular_constraint requests: the outlines index when the package is there, else the grammar matcher
            import outlines_core  # noqa: F401

            return OutlinesConstraintBackend
        except Exception:
            return XgrammarBackend
    if getattr(args, "first_token_constraint_mode", False):
        return FirstTokenConstraintBackend
    if getattr(args, "diverse_mode", False):
        return DiverseBackend
    return ModelBackend
