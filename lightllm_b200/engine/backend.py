"""The per-GPU inference backend: turns the request table into prefill / decode forward passes,
samples, and publishes results into the shared request objects.

One backend per model-rank process.  All TP ranks of a replica run the same deterministic
schedule on the same request list, so they stay in lock step without exchanging decisions;
with data-parallel attention (`dp > 1`) replicas exchange only their (prefill, decode) counts
per step and pad idle replicas with the HOLD request.

Step anatomy (chunked prefill, the default mode):
    classify -> [pause if the pool is short] -> prefill chunk(s) OR one decode step
    -> sample on device -> token ids stay on device for the next decode (scatter into the request
    table's next-token column) and are copied to pinned host memory for stop checks / detokenizer.

Reference: lightllm/server/router/model_infer/mode_backend/base_backend.py (ModeBackend),
chunked_prefill/impl.py (ChunkedPrefillBackend), generic_pre_process.py, generic_post_process.py.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import numpy as np
import torch

from .. import ops
from ..common.infer_state import ModelInput
from ..server.core.objs.req import FinishStatus, Req
from .infer_batch import InferenceContext, InferReq
from .native_radix import NativeRadixCache as RadixCache


@dataclass
class BackendArgs:
    batch_max_tokens: int = 16384
    chunked_prefill_size: int = 8192
    disable_chunked_prefill: bool = False
    router_max_wait_tokens: int = 1
    disable_aggressive_schedule: bool = False
    disable_dynamic_prompt_cache: bool = False
    eos_ids: tuple = ()
    max_req_total_len: int = 8192
    return_all_prompt_logprobs: bool = False
    enable_prefill_decode_mixed: bool = False
    pause_recover_interval: int = 100
    cpu_cache_bytes: int = 0          # > 0: second prefix-cache tier in pinned host memory
    cpu_cache_page_tokens: int = 256
    disk_cache_dir: Optional[str] = None
    disk_cache_bytes: int = 0
    # decode steps are launched before the previous step's tokens have been read back: the host-side bookkeeping
    # of step k (token append, finish checks, publishing) runs while the GPU executes step k + 1
    enable_decode_overlap: bool = True
    linear_att_hash_page_size: int = 512   # hybrid models: token granularity of the recurrent-state snapshots
    state_host_cache_bytes: int = 0        # hybrid models: pinned host room for snapshots pushed out of the GPU table


class PinnedRing:
    """A few pinned host buffers per key used round-robin, so an async copy issued for step k is not
    overwritten while step k+1 is prepared (reference: pin_mem_manager.py)."""

    def __init__(self, depth: int = 4, pin: bool = True):
        self.depth = depth
        self.pin = pin and torch.cuda.is_available()
        self._bufs: Dict[str, list] = {}
        self._i: Dict[str, int] = {}

    def get(self, key: str, n: int, dtype) -> torch.Tensor:
        lst = self._bufs.setdefault(key, [None] * self.depth)
        i = self._i.get(key, 0)
        self._i[key] = (i + 1) % self.depth
        b = lst[i]
        if b is None or b.numel() < n or b.dtype != dtype:
            b = torch.empty(max(n, 1024), dtype=dtype, pin_memory=self.pin)
            lst[i] = b
        return b[:n]

    def from_numpy(self, key: str, arr: np.ndarray, dtype) -> torch.Tensor:
        t = self.get(key, arr.shape[0], dtype)
        t.numpy()[:] = arr
        return t


class ControlState:
    """Prefill-vs-decode choice: aggressive = prefill whenever something waits; otherwise at most one
    prefill per `router_max_wait_tokens` decode steps (reference: control_state.py)."""

    def __init__(self, args: BackendArgs):
        self.aggressive = not args.disable_aggressive_schedule
        self.max_wait = args.router_max_wait_tokens
        self.decode_since_prefill = 0
        self.step = 0

    def select(self, n_prefill: int, n_decode: int) -> str:
        self.step += 1
        if n_prefill == 0 and n_decode == 0:
            return "idle"
        if n_prefill == 0:
            self.decode_since_prefill += 1
            return "decode"
        if n_decode == 0 or self.aggressive or self.decode_since_prefill >= self.max_wait:
            self.decode_since_prefill = 0
            return "prefill"
        self.decode_since_prefill += 1
        return "decode"


class ModelBackend:
    def __init__(self, model, args: Optional[BackendArgs] = None, is_master_in_dp: bool = True,
                 on_token: Optional[Callable[[InferReq, int, float], None]] = None):
        self.model = model
        self.args = args or BackendArgs()
        self.device = model.device
        state_slots = int(getattr(model, "state_snapshot_slots", 0) or 0)
        if not getattr(model, "supports_prefix_cache", True) and state_slots <= 0:
            # hybrid models keep per-request recurrent state: without state snapshots a shared prefix is useless
            self.args.disable_dynamic_prompt_cache = True
        self.radix_cache = None if self.args.disable_dynamic_prompt_cache else \
            RadixCache("radix", model.max_total_token_num, 0, model.mem_manager)
        self.ctx = InferenceContext(model, self.radix_cache)
        self.state_cache = None
        if self.radix_cache is not None and not getattr(model, "supports_prefix_cache", True):
            from .state_cache import StateSnapshotCache

            self.state_cache = StateSnapshotCache(model, self.args.linear_att_hash_page_size,
                                                  host_bytes=self.args.state_host_cache_bytes)
            self.ctx.state_cache = self.state_cache
        if self.args.cpu_cache_bytes > 0 and self.radix_cache is not None and self.state_cache is None:
            from .host_kv_cache import HostKVCache

            self.ctx.host_cache = HostKVCache(model.mem_manager, self.args.cpu_cache_bytes,
                                              self.args.cpu_cache_page_tokens, self.args.disk_cache_dir,
                                              self.args.disk_cache_bytes, name=f"rank{model.ps.global_rank}")
        on = os.environ.get("LLB_RADIX_TREE_MERGE_ENABLE", os.environ.get("LIGHTLLM_RADIX_TREE_MERGE_ENABLE", ""))
        self._merge_delta = int(os.environ.get("LLB_RADIX_TREE_MERGE_DELTA", os.environ.get(
            "LIGHTLLM_RADIX_TREE_MERGE_DELTA", "6000"))) if on.strip().upper() in ("1", "ON", "TRUE") else 0
        self._merge_ticks = 0
        self.pins = PinnedRing(pin=self.device.type == "cuda")
        self.control = ControlState(self.args)
        self.is_master_in_dp = is_master_in_dp   # only one rank per replica writes into shm
        self.on_token = on_token
        self.eos_ids = set(self.args.eos_ids)
        self.prefill_mask_func = None   # hooks for constrained decoding backends
        self.decode_mask_func = None
        self.extra_post_req_handle_func = None
        self.stats = {"prefill_steps": 0, "decode_steps": 0, "prefill_tokens": 0, "decode_tokens": 0,
                      "h2d_bytes": 0, "d2h_bytes": 0, "paused": 0}
        self._steps = 0
        self._step_timing = os.environ.get("LLB_STEP_TIMING", "0") == "1"
        self._pending = None  # a launched decode step whose tokens have not been read back yet
        if self.radix_cache is not None and model.config.get("prompt_cache_kv_buffer"):
            self.preload_prompt_cache_kv(model.config, getattr(model, "model_dir", None))

    # ------------------------------------------------------------------ saved prompt prefix
    def save_prompt_cache_kv(self, token_ids, path: str) -> int:
        """Writes the KV rows of a cached prompt prefix (as they sit in the pool: every layer's rows of this rank's KV
        heads) to `path`; returns the number of tokens saved.  A deployment lists the file per rank under
        `prompt_cache_kv_buffer` and the tokens under `prompt_cache_token_ids` in config.json; at start-up the rows
        are loaded into the pool and pinned in the prefix tree (a system prompt computed once, e.g. in full precision
        for a quantised deployment).  Reference: lightllm/server/router/model_infer/infer_batch.py:253-265."""
        ids = np.asarray(token_ids, dtype=np.int64)
        node, n, slots = self.radix_cache.match_prefix(ids, update_refs=True)
        if node is None:
            return 0
        try:
            pages = self.model.mem_manager.gather_pages(torch.from_numpy(np.ascontiguousarray(slots[:n])).to(torch.int32))
            torch.save({"token_ids": torch.from_numpy(ids[:n].copy()), "kv": pages.cpu()}, path)
        finally:
            self.radix_cache.dec_node_ref_counter(node)
        return n

    def preload_prompt_cache_kv(self, cfg: dict, model_dir: Optional[str]) -> int:
        """Loads the saved prefix of this rank and pins it (reference:
        lightllm/server/router/model_infer/mode_backend/base_backend.py:961-977)."""
        rank = self.model.ps.global_rank
        files = cfg["prompt_cache_kv_buffer"]
        name = files.get(f"rank_{rank}") if isinstance(files, dict) else files
        if not name:
            return 0
        path = name if os.path.isabs(name) or not model_dir else os.path.join(model_dir, name)
        blob = torch.load(path, weights_only=True, map_location="cpu")
        kv = blob["kv"] if isinstance(blob, dict) else blob
        ids = np.asarray(cfg.get("prompt_cache_token_ids") if cfg.get("prompt_cache_token_ids") is not None
                         else blob["token_ids"], dtype=np.int64)
        mm = self.model.mem_manager
        n = min(len(ids), kv.shape[1])
        want = (mm.layer_num, *mm.kv_row_shape())
        if (kv.shape[0], *kv.shape[2:]) != want or kv.dtype != mm.dtype:
            raise ValueError(f"prompt cache file {path}: rows {tuple(kv.shape)} {kv.dtype} do not fit this pool "
                             f"{want} {mm.dtype}")
        slots = mm.alloc(n).clone()
        mm.scatter_pages(slots, kv[:, :n].to(mm.device))
        self.radix_cache.insert(ids[:n], slots.cpu().numpy().astype(np.int32))
        self.radix_cache.match_prefix(ids[:n], update_refs=True)       # pinned for the life of the process
        self.stats["prompt_cache_preloaded_tokens"] = n
        return n

    # ------------------------------------------------------------------ requests
    def add_reqs(self, shm_reqs: List[Req]) -> List[InferReq]:
        out = []
        for r in shm_reqs:
            req = self.ctx.add_req(r)
            if req is None:
                raise RuntimeError("request table full: running_max_req_size must not exceed the model's max_req_num")
            out.append(req)
        return out

    def fetch_prefixes(self, new_reqs) -> int:
        """Data-parallel serving: pulls the part of each new prompt that another replica has cached and this one has
        not (`engine/dp_prefix_fetch.py`).  `new_reqs` = (owner replica, prompt ids) of every new request, the same
        list on every rank; collective."""
        if getattr(self, "_prefix_fetch", None) is None:
            from .dp_prefix_fetch import DPPrefixFetch

            self._prefix_fetch = DPPrefixFetch(self)
        n = self._prefix_fetch.run(new_reqs)
        self.stats["dp_fetched_tokens"] = self.stats.get("dp_fetched_tokens", 0) + n
        return n

    def abort(self, req_id: int):
        req = self.ctx.requests.get(req_id)
        if req is not None:
            req.infer_aborted = True

    def stop_str_matched(self, req_id: int):
        req = self.ctx.requests.get(req_id)
        if req is not None:
            req.stop_str_matched = True

    def has_work(self) -> bool:
        return bool(self.ctx.requests) or self._pending is not None

    # ------------------------------------------------------------------ classification
    def _get_classed_reqs(self):
        """Splits live requests into (prefill list with chunk sizes, decode list); finishes aborted ones;
        pauses requests when the pool cannot serve the step."""
        ctx, a = self.ctx, self.args
        prefill, decode, finished = [], [], []
        budget = a.batch_max_tokens
        chunk_cap = a.batch_max_tokens if a.disable_chunked_prefill else a.chunked_prefill_size
        can_alloc = ctx.get_can_alloc_token_num()
        recover = (self._steps % a.pause_recover_interval == 0)
        paused_now = 0
        for rid in ctx.infer_req_ids:
            req = ctx.requests[rid]
            if req.finish_status.is_finished():
                finished.append(req)
                continue
            # `infer_aborted` is only ever set by abort(), which the rank process calls when an AbortedReqCmd
            # arrives through the mailbox whose generation all tensor-parallel ranks agree on.  The shared
            # request's own `is_aborted` flag is written by the HTTP worker at an arbitrary moment: ranks whose
            # loops are a step apart would drop the request at different steps and run batches of different
            # sizes (reference: base_backend.py:543-546 sets infer_aborted from the command as well).
            if req.infer_aborted or req.stop_str_matched:
                self._finish_without_token(req)
                finished.append(req)
                continue
            if req.paused:
                if recover and can_alloc > req.total_len() + 64:
                    ctx.recover_req(req)
                else:
                    continue
            if req.inflight:
                # its last token is still on the device: it decodes on unless that token must be its last
                out = req.cur_output_len + req.inflight
                if out >= req.sampling.max_new_tokens or req.shm_req.input_len + out >= a.max_req_total_len:
                    continue
            if not req.inflight and req.need_prefill():
                remaining = req.total_len() - req.cur_kv_len
                chunk = min(remaining, chunk_cap)
                if self.state_cache is not None:
                    # end a chunk at the last page boundary of the prompt: the state there is worth keeping
                    page = self.state_cache.page
                    last = (req.total_len() - 1) // page * page
                    if req.cur_kv_len < last < req.cur_kv_len + chunk:
                        chunk = last - req.cur_kv_len
                if chunk <= budget and chunk <= can_alloc:
                    prefill.append((req, chunk))
                    budget -= chunk
                    can_alloc -= chunk
            else:
                if can_alloc >= 1:
                    decode.append(req)
                    can_alloc -= 1
                elif paused_now < 2:  # pool exhausted: pause (at most two per step), re-prefill later
                    ctx.pause_req(req)
                    paused_now += 1
                    self.stats["paused"] += 1
                    can_alloc = ctx.get_can_alloc_token_num()
        return prefill, decode, finished

    def _finish_without_token(self, req: InferReq):
        """Aborted / stop-string requests end with a synthetic final token so downstream stages drain."""
        status = FinishStatus.FINISHED_ABORTED if req.infer_aborted else FinishStatus.FINISHED_STOP
        if req.cur_output_len == 0 or req.infer_aborted:
            eos = next(iter(self.eos_ids)) if self.eos_ids else 0
            req.append_token(eos, 0.0)
        req.finish_status.set_status(status)
        if self.is_master_in_dp:
            req.publish()

    # ------------------------------------------------------------------ one step
    @torch.no_grad()
    def _tick_tree_merge(self):
        """`LIGHTLLM_RADIX_TREE_MERGE_ENABLE=1`: every `LIGHTLLM_RADIX_TREE_MERGE_DELTA` (default 6000) forward
        passes the prefix tree merges its chains of unreferenced single-child nodes.  The tick counts forward
        passes, which the ranks of a tensor-parallel group run in lock-step, so their trees stay identical.
        Reference: mode_backend/base_backend.py:620-632."""
        if self._merge_delta <= 0 or self.radix_cache is None:
            return
        self._merge_ticks += 1
        if self._merge_ticks % self._merge_delta == 0:
            self.tree_merges = getattr(self, "tree_merges", 0) + int(self.radix_cache.merge_unreferenced_nodes() or 0)

    def step(self) -> dict:
        """Runs at most one forward pass.  Returns {"kind", "finished": [InferReq], "tokens": n}."""
        self._steps += 1
        fused = getattr(self.model.tp, "fused", None)
        if fused is not None and (self._steps & 127) == 1:
            fused.check()
        if (self._steps & 127) == 1 and getattr(self.model, "debug_status", None) is not None:
            self.model.check_debug_bounds()
        prefill, decode, finished = self._get_classed_reqs()
        kind = self.control.select(len(prefill), len(decode))
        n_tok = 0
        if kind == "decode" and self._can_defer(decode):
            n_tok = self._run_decode(decode, defer=True)   # launches step k + 1, then settles step k
        else:
            if self._pending is not None:  # settle the step in flight, then look at the requests again
                self._flush_pending()
                prefill, decode, fin2 = self._get_classed_reqs()
                finished += [r for r in fin2 if r not in finished]
                kind = self.control.select(len(prefill), len(decode))
            if kind == "prefill":
                n_tok = self._run_prefill(prefill)
            elif kind == "decode":
                n_tok = self._run_decode(decode)
        if kind in ("prefill", "decode"):
            self._tick_tree_merge()
        for req in list(self.ctx.requests.values()):
            if req.finish_status.is_finished() and req not in finished:
                finished.append(req)
        finished = [r for r in finished if not r.retire_hold]   # e.g. prompt KV still being sent to a decode node
        for req in finished:
            self.ctx.remove_req(req)
        return {"kind": kind, "finished": finished, "tokens": n_tok}

    # ---- prefill ----
    def _run_prefill(self, items) -> int:
        reqs = [r for r, _ in items]
        B = len(reqs)
        chunks = np.array([c for _, c in items], dtype=np.int32)
        ready = np.array([r.cur_kv_len for r in reqs], dtype=np.int32)
        total = int(chunks.sum())
        ids = np.concatenate([r.get_chunked_input_token_ids(int(c)) for r, c in items])
        slots = self.ctx.alloc_slots(total)
        slots_np = slots.numpy()
        off = 0
        for r, c in items:
            r.slots = np.concatenate([r.slots[: r.cur_kv_len], slots_np[off:off + c]])
            off += int(c)
        pin = self.pins
        want_all = self.args.return_all_prompt_logprobs and any(r.sampling.prompt_logprobs >= 0 for r in reqs)
        mm = None
        if any(getattr(r.shm_req, "_mm_params", None) for r in reqs):
            mm = []
            for r in reqs:
                p = getattr(r.shm_req, "_mm_params", None)
                if p and getattr(self.model, "needs_prompt_ids", False):
                    p = dict(p)
                    p["_prompt_ids"] = np.asarray(r.shm_req.shm_prompt_ids.arr[: r.shm_req.input_len])
                mm.append(p)
        mi = ModelInput(batch_size=B, total_token_num=int((ready + chunks).sum()), max_kv_len=int((ready + chunks).max()),
                        is_prefill=True,
                        b_req_idx=pin.from_numpy("p_req", np.array([r.req_idx for r in reqs], dtype=np.int32), torch.int32),
                        b_seq_len=pin.from_numpy("p_seq", ready + chunks, torch.int32),
                        mem_indexes=slots,
                        input_ids=pin.from_numpy("p_ids", ids.astype(np.int64), torch.int64),
                        b_ready_cache_len=pin.from_numpy("p_ready", ready, torch.int32),
                        b_q_len=pin.from_numpy("p_qlen", chunks, torch.int32), max_q_len=int(chunks.max()),
                        return_all_logits=want_all, multimodal_params=mm)
        self.stats["h2d_bytes"] += total * 8 + total * 4 + B * 16
        out = self.model.forward(mi)
        has_out = np.array([r.cur_kv_len + int(c) >= r.total_len() for r, c in items], dtype=bool)
        for r, c in items:
            r.cur_kv_len += int(c)
        self._snapshot_states(reqs)
        logits = out.logits if want_all else self._logits_for_sampling(out, reqs, is_prefill=True)
        if want_all:
            self._handle_prompt_logprobs(reqs, chunks, ids, logits)
            last_rows = torch.from_numpy(np.cumsum(chunks) - 1).to(self.device)
            logits = logits.index_select(0, last_rows)
        if has_out.any():
            self._sample_and_post(reqs, logits, has_out, is_prefill=True)
        elif self.is_master_in_dp:
            for r in reqs:
                r.shm_req.shm_cur_kv_len = r.cur_kv_len
        self.stats["prefill_steps"] += 1
        self.stats["prefill_tokens"] += total
        return int(has_out.sum())

    def _handle_prompt_logprobs(self, reqs, chunks, ids, logits):
        """logprob of every prompt token given its prefix, written beside the prompt ids."""
        T = ids.shape[0]
        nxt = np.empty(T, dtype=np.int64)
        off = 0
        for r, c in zip(reqs, chunks):
            c = int(c)
            start = r.cur_kv_len - c  # cur_kv_len already advanced
            arr = r.shm_req.shm_prompt_ids.arr
            nxt[off:off + c] = arr[start + 1:start + c + 1]
            off += c
        nxt_dev = torch.from_numpy(nxt).to(self.device)
        lp = ops.token_logprob(logits, nxt_dev).cpu().numpy()
        off = 0
        for r, c in zip(reqs, chunks):
            c = int(c)
            start = r.cur_kv_len - c
            n = min(c, r.shm_req.input_len - 1 - start)
            if n > 0 and self.is_master_in_dp:
                r.shm_req.shm_logprobs.arr[start + 1:start + 1 + n] = lp[off:off + n]
                meta = getattr(r.shm_req, "shm_prompt_meta", None)
                if meta is not None and r.sampling.prompt_logprobs >= 0:
                    self._prompt_rank_and_topk(meta.arr, start, n, logits[off:off + n], nxt_dev[off:off + n])
            off += c

    @staticmethod
    def _prompt_rank_and_topk(out: np.ndarray, start: int, n: int, logits, next_ids, block: int = 1024):
        """Rank of every prompt token among the vocabulary at its position and the k most likely tokens there
        (out[pos] = [rank, k ids, k logprobs]); in blocks of rows, the log-softmax of a block is materialised."""
        k = (out.shape[1] - 1) // 2
        for a in range(0, n, block):
            b = min(a + block, n)
            lsm = torch.log_softmax(logits[a:b].float(), dim=-1)
            own = lsm.gather(1, next_ids[a:b].view(-1, 1))
            rank = (lsm > own).sum(-1) + 1
            rows = slice(start + 1 + a, start + 1 + b)
            out[rows, 0] = rank.float().cpu().numpy()
            if k:
                vals, idx = lsm.topk(k, dim=-1)
                out[rows, 1:1 + k] = idx.float().cpu().numpy()
                out[rows, 1 + k:] = vals.cpu().numpy()

    # ---- decode ----
    def _snapshot_states(self, reqs: List[InferReq]):
        """Hybrid models: keep the recurrent state of every request that now stands at a page boundary."""
        sc = self.state_cache
        if sc is None:
            return
        for r in reqs:
            n = r.cur_kv_len
            if n > 0 and n % sc.page == 0 and not r.shm_req.sample_params.disable_prompt_cache:
                sc.save(r.req_idx, r.shm_req.shm_prompt_ids.arr[:n])

    def _can_defer(self, reqs: List[InferReq]) -> bool:
        """A decode step may be launched ahead of the previous step's bookkeeping when nothing on the host shapes its
        logits (penalties, token masks, constrained decoding) and this is the plain backend."""
        on_gpu = self.device.type == "cuda" or os.environ.get("LLB_FORCE_DECODE_OVERLAP") == "1"  # CPU: tests only
        if not (self.args.enable_decode_overlap and on_gpu and type(self).__name__ in ("ModelBackend", "DPBackend")):
            return False
        if self.state_cache is not None:   # snapshots are taken between steps
            return False
        if self.decode_mask_func is not None or self.extra_post_req_handle_func is not None:
            return False
        for r in reqs:
            sp = r.sampling
            if sp.has_penalty or sp.invalid_token_ids or sp.allowed_token_ids or sp.exp_decay_factor > 1.0 or \
                    (self.eos_ids and not sp.ignore_eos and r.cur_output_len + r.inflight + 1 < sp.min_new_tokens):
                return False
        return True

    def _flush_pending(self):
        """Reads back the tokens of the decode step in flight and does its host-side bookkeeping."""
        pend, self._pending = self._pending, None
        if pend is None:
            return
        reqs, ids_h, lps_h, event = pend
        if event is not None:
            t0 = time.perf_counter()
            event.synchronize()
            self.stats["wait_gpu_s"] = self.stats.get("wait_gpu_s", 0.0) + (time.perf_counter() - t0)
        live = []
        for i, r in enumerate(reqs):
            r.inflight = 0
            # a request that ended in the meantime (its previous token was an end token) drops this extra token
            live.append(not r.finish_status.is_finished())
        self._post(reqs, ids_h.numpy(), lps_h.numpy(), np.array(live, dtype=bool))

    def _run_decode(self, reqs: List[InferReq], defer: bool = False) -> int:
        B = len(reqs)
        slots = self.ctx.alloc_slots(B)
        slots_np = slots.numpy()
        seq = np.empty(B, dtype=np.int32)
        idx = np.empty(B, dtype=np.int32)
        for i, r in enumerate(reqs):
            r.slots = np.append(r.slots[: r.cur_kv_len], slots_np[i])
            r.cur_kv_len += 1
            seq[i] = r.cur_kv_len
            idx[i] = r.req_idx
        pin = self.pins
        mi = ModelInput(batch_size=B, total_token_num=int(seq.sum()), max_kv_len=int(seq.max()), is_prefill=False,
                        b_req_idx=pin.from_numpy("d_req", idx, torch.int32),
                        b_seq_len=pin.from_numpy("d_seq", seq, torch.int32), mem_indexes=slots)
        self.stats["h2d_bytes"] += B * 12
        timing = self._step_timing and not defer and self.device.type == "cuda"
        if timing:   # LLB_STEP_TIMING=1: device time of the synchronous decode passes (forward + sampling)
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        out = self.model.forward(mi)
        if defer:
            ids, lps = self._sample(reqs, self._logits_for_sampling(out, reqs, False), np.ones(B, dtype=bool),
                                    is_prefill=False)
            if self.device.type == "cuda":
                ids_h = self.pins.get("s_ids", B, torch.int64)
                lps_h = self.pins.get("s_lps", B, torch.float32)
                ids_h.copy_(ids, non_blocking=True)
                lps_h.copy_(lps, non_blocking=True)
                event = torch.cuda.Event()
                event.record(torch.cuda.current_stream(self.device))
            else:
                ids_h, lps_h, event = ids.clone(), lps.clone(), None
            self.stats["d2h_bytes"] += B * 12
            prev, self._pending = self._pending, None
            if prev is not None:  # the previous step's bookkeeping overlaps this step's execution
                self._pending = prev
                self._flush_pending()
            for r in reqs:
                r.inflight = 1
            self._pending = (reqs, ids_h, lps_h, event)
        else:
            self._snapshot_states(reqs)
            if timing:
                ids, lps = self._sample(reqs, self._logits_for_sampling(out, reqs, False), np.ones(B, dtype=bool), False)
                ev1.record()
                self._post_sampled(reqs, ids, lps, np.ones(B, dtype=bool))
                self.stats["decode_gpu_ms"] = self.stats.get("decode_gpu_ms", 0.0) + ev0.elapsed_time(ev1)
            else:
                self._sample_and_post(reqs, self._logits_for_sampling(out, reqs, False), np.ones(B, dtype=bool),
                                      is_prefill=False)
        self.stats["decode_steps"] += 1
        self.stats["decode_tokens"] += B
        return B

    # ---- sampling + post ----
    sharded_sampling = True   # subclasses that read whole logit rows in their own sampling code turn this off

    def _needs_full_rows(self, reqs: List[InferReq], is_prefill: bool) -> bool:
        if (self.prefill_mask_func if is_prefill else self.decode_mask_func) is not None:
            return True
        for r in reqs:
            sp = r.sampling
            if sp.top_k != 1 or sp.has_penalty or sp.invalid_token_ids or sp.allowed_token_ids or \
                    sp.exp_decay_factor > 1.0 or \
                    (self.eos_ids and not sp.ignore_eos and r.cur_output_len + r.inflight + 1 < sp.min_new_tokens):
                return True
        return False

    def _logits_for_sampling(self, out, reqs: List[InferReq], is_prefill: bool):
        """The model's vocabulary shards when this step can be sampled from them (tensor parallelism, every row
        greedy, nothing that edits logit rows), else the dense matrix."""
        x = out.logits_any
        if x is None or isinstance(x, torch.Tensor):
            return x
        if self.sharded_sampling and not self._needs_full_rows(reqs, is_prefill):
            return x
        return out.logits

    def _sample(self, reqs: List[InferReq], logits: torch.Tensor, has_out: np.ndarray, is_prefill: bool):
        """Masks / penalties, sampling and the device-side hand-over of the sampled ids to the next decode step."""
        dev = self.device
        sp = [r.sampling for r in reqs]
        mask_func = self.prefill_mask_func if is_prefill else self.decode_mask_func
        if isinstance(logits, torch.Tensor):   # vocabulary shards only get here when nothing edits the rows
            if mask_func is not None:
                mask_func(reqs, logits)
            self._apply_penalties(reqs, logits)
        all_greedy = all(s.top_k == 1 for s in sp)
        if all_greedy:
            ids, lps = ops.sample(logits)
        else:
            temp = torch.tensor([s.temperature for s in sp], dtype=torch.float32).to(dev, non_blocking=True)
            top_p = torch.tensor([s.top_p for s in sp], dtype=torch.float32).to(dev, non_blocking=True)
            top_k = torch.tensor([s.top_k for s in sp], dtype=torch.int32).to(dev, non_blocking=True)
            seeds = torch.tensor([r.seed for r in reqs], dtype=torch.int64).to(dev, non_blocking=True)
            steps = torch.tensor([r.cur_output_len + r.inflight for r in reqs], dtype=torch.int64).to(dev, non_blocking=True)
            ids, lps = ops.sample(logits, temp, top_p, top_k, seeds, steps)
        # the next decode step reads its input ids on the device
        b_req_idx = torch.tensor([r.req_idx for r in reqs], dtype=torch.int32).to(dev, non_blocking=True)
        has_dev = None if has_out.all() else torch.from_numpy(has_out.astype(np.uint8)).to(dev, non_blocking=True)
        ops.scatter_next_token_(self.model.req_manager.req_to_next_token_ids, ids, b_req_idx, has_dev)
        return ids, lps

    def _sample_and_post(self, reqs: List[InferReq], logits: torch.Tensor, has_out: np.ndarray, is_prefill: bool):
        ids, lps = self._sample(reqs, logits, has_out, is_prefill)
        self._post_sampled(reqs, ids, lps, has_out)

    def _post_sampled(self, reqs: List[InferReq], ids, lps, has_out: np.ndarray):
        dev = self.device
        B = len(reqs)
        if dev.type == "cuda":
            ids_h = self.pins.get("s_ids", B, torch.int64)
            lps_h = self.pins.get("s_lps", B, torch.float32)
            ids_h.copy_(ids, non_blocking=True)
            lps_h.copy_(lps, non_blocking=True)
            torch.cuda.current_stream(dev).synchronize()
        else:
            ids_h, lps_h = ids, lps
        self.stats["d2h_bytes"] += B * 12
        self._post(reqs, ids_h.numpy(), lps_h.numpy(), has_out)

    def _dump_routed_experts(self, r: InferReq):
        """Copies the routed expert ids of the request's tokens (all but the last produced one, which never went
        through the model) into the request's shared array.  Reference:
        lightllm/server/router/model_infer/infer_req_ext.py:177-192."""
        sr = r.shm_req
        out = getattr(sr, "shm_routed", None)
        if out is None:
            return
        n = min(r.cur_kv_len, sr.input_len + r.cur_output_len - 1, out.arr.shape[0])
        if n <= 0:
            return
        slots = self.model.req_manager.req_to_token_indexs[r.req_idx, :n]
        out.arr[:n] = self.model.route_capture.extract(slots)
        sr.routed_len = n

    def _post(self, reqs: List[InferReq], ids_np, lps_np, has_out):
        """Host-side bookkeeping of sampled tokens: append, finish checks, publishing to the shared request."""
        now = time.time()
        for i, r in enumerate(reqs):
            if not has_out[i]:
                if self.is_master_in_dp and not r.finish_status.is_finished():
                    r.shm_req.shm_cur_kv_len = r.cur_kv_len
                continue
            tok = int(ids_np[i])
            r.append_token(tok, float(lps_np[i]))
            r.update_finish_status(self.eos_ids, self.args.max_req_total_len)
            if self.extra_post_req_handle_func is not None:
                self.extra_post_req_handle_func(r, tok, float(lps_np[i]))
            if self.is_master_in_dp and not r.retire_hold:
                if r.cur_output_len == 1:
                    r.shm_req.first_token_time = now
                if r.finish_status.is_finished() and getattr(self.model, "route_capture", None) is not None:
                    self._dump_routed_experts(r)      # before the finish state becomes visible
                r.publish()
            if self.on_token is not None:
                self.on_token(r, tok, float(lps_np[i]))

    def _apply_penalties(self, reqs: List[InferReq], logits: torch.Tensor):
        """Builds the CSR (token id, count) lists of the requests that use penalties, the masks of
        invalid / not-yet-allowed tokens (eos before min_new_tokens), and applies them in one kernel."""
        need_pen = any(r.sampling.has_penalty for r in reqs)
        need_mask = any(r.sampling.invalid_token_ids or
                        (self.eos_ids and not r.sampling.ignore_eos
                         and r.cur_output_len + 1 < r.sampling.min_new_tokens)
                        for r in reqs)
        need_decay = any(r.sampling.exp_decay_factor > 1.0 for r in reqs)
        for i, r in enumerate(reqs):      # `allowed_token_ids`: everything else becomes impossible (rare: torch ops)
            if r.sampling.allowed_token_ids:
                ok = torch.tensor([t for t in r.sampling.allowed_token_ids if 0 <= t < logits.shape[1]],
                                  dtype=torch.long, device=logits.device)
                keep = logits[i, ok].clone()
                logits[i].fill_(float("-inf"))
                logits[i, ok] = keep
        if not (need_pen or need_mask or need_decay):
            return
        dev = self.device
        B = len(reqs)
        cu = mask_cu = tok_ids = tok_cnt = mask_ids = pres = freq = rep = None
        if need_pen:
            cu_l, ids_l, cnt_l = [0], [], []
            for r in reqs:
                if r.sampling.has_penalty:
                    ids_l.extend(r.out_token_counter.keys())
                    cnt_l.extend(r.out_token_counter.values())
                cu_l.append(len(ids_l))
            cu = torch.tensor(cu_l, dtype=torch.int32).to(dev)
            tok_ids = torch.tensor(ids_l or [0], dtype=torch.int32).to(dev)
            tok_cnt = torch.tensor(cnt_l or [0], dtype=torch.int32).to(dev)
            pres = torch.tensor([r.sampling.presence_penalty for r in reqs], dtype=torch.float32).to(dev)
            freq = torch.tensor([r.sampling.frequency_penalty for r in reqs], dtype=torch.float32).to(dev)
            rep = torch.tensor([r.sampling.repetition_penalty for r in reqs], dtype=torch.float32).to(dev)
        if need_mask:
            mcu, mids = [0], []
            for r in reqs:
                mids.extend(r.sampling.invalid_token_ids)
                if r.cur_output_len + 1 < r.sampling.min_new_tokens and not r.sampling.ignore_eos:
                    mids.extend(self.eos_ids)
                mcu.append(len(mids))
            mask_cu = torch.tensor(mcu, dtype=torch.int32).to(dev)
            mask_ids = torch.tensor(mids or [0], dtype=torch.int32).to(dev)
        if need_decay and self.eos_ids:
            # exponential_decay_length_penalty: eos logit scaled up as the output grows past `start`
            eos = sorted(self.eos_ids)
            for i, r in enumerate(reqs):
                f, s = r.sampling.exp_decay_factor, r.sampling.exp_decay_start
                if f > 1.0 and r.cur_output_len > s:
                    scale = f ** (r.cur_output_len - s)
                    row = logits[i, eos]
                    logits[i, eos] = torch.where(row > 0, row * scale, row / scale)
        if need_pen or need_mask:
            ops.apply_penalty_(logits, pres, freq, rep, cu, tok_ids, tok_cnt, mask_cu, mask_ids)
