"""Per-rank runtime state of requests and the resource bookkeeping around them.

`InferReq` mirrors one shm `Req` inside a model-rank process: how much of it is in the KV pool,
which pool slots it owns (kept on the host, they come from the host-side allocator), the radix
node it shares a prefix with, and its sampling state.  `InferenceContext` owns the request
table: admission (slot allocation + radix match), release (donate KV to the radix tree, free
the rest), pause / recover under memory pressure.

Reference: lightllm/server/router/model_infer/infer_batch.py (InferenceContext :31-437,
InferReq :502-922, InferReqUpdatePack :935-991).
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import numpy as np
import torch

from ..server.core.objs.req import FinishStatus, Req


class InferSamplingParams:
    """Unpacked, read-only view of the request's SamplingParams for the hot loop."""

    __slots__ = ("do_sample", "presence_penalty", "frequency_penalty", "repetition_penalty", "temperature", "top_p",
                 "top_k", "ignore_eos", "max_new_tokens", "min_new_tokens", "stop_sequences", "seed", "has_penalty",
                 "exp_decay_start", "exp_decay_factor", "invalid_token_ids", "allowed_token_ids", "input_penalty",
                 "regular_constraint", "guided_grammar", "guided_json", "prompt_logprobs")

    def __init__(self, sp, vocab_size: int):
        self.do_sample = sp.do_sample
        self.presence_penalty = sp.presence_penalty
        self.frequency_penalty = sp.frequency_penalty
        self.repetition_penalty = sp.repetition_penalty
        self.temperature = sp.temperature
        self.top_p = sp.top_p
        self.top_k = sp.top_k if sp.top_k > 0 else vocab_size
        self.ignore_eos = sp.ignore_eos
        self.max_new_tokens = sp.max_new_tokens
        self.min_new_tokens = sp.min_new_tokens
        self.stop_sequences = [s for s in sp.stop_sequences.to_list() if s]
        self.seed = sp.seed
        self.exp_decay_start, self.exp_decay_factor = sp.exponential_decay_length_penalty.to_tuple()
        self.invalid_token_ids = sp.invalid_token_ids.to_list()
        self.allowed_token_ids = sp.allowed_token_ids.to_list()
        self.input_penalty = sp.input_penalty
        self.regular_constraint = sp.regular_constraint.get() or None
        self.guided_grammar = sp.guided_grammar.get() or None
        self.guided_json = sp.guided_json.get() or None
        self.prompt_logprobs = sp.prompt_logprobs
        self.has_penalty = (self.presence_penalty != 0.0 or self.frequency_penalty != 0.0
                            or self.repetition_penalty != 1.0)


class InferReq:
    def __init__(self, shm_req: Req, req_idx: int, vocab_size: int, dp_index: int = 0):
        self.shm_req = shm_req
        self.req_id = shm_req.request_id
        self.req_idx = req_idx                 # row in req_to_token_indexs
        self.sampling = InferSamplingParams(shm_req.sample_params, vocab_size)
        self.cur_kv_len = 0                    # tokens whose KV is in the pool
        self.cur_output_len = shm_req.shm_cur_output_len
        self.slots = np.empty(0, dtype=np.int32)  # pool slot of every cached position (host mirror)
        self.shared_kv_node = None             # radix node referenced by this request
        self.shared_len = 0                    # leading tokens owned by the radix tree
        self.finish_status = FinishStatus()
        self.infer_aborted = False
        self.stop_str_matched = False
        self.paused = False
        self.inflight = 0                      # decode steps launched whose token has not been read back yet
        self.retire_hold = False               # finished but not to be published / removed yet (KV transfer running)
        self.filter_mark = False
        self.out_token_counter: Dict[int, int] = {}
        self.cumlogprob = 0.0
        # sub-requests of one group (n > 1) share the user's seed: offset it by the index inside the group
        self.seed = (self.sampling.seed + (self.req_id - shm_req.group_req_id)) if self.sampling.seed >= 0 \
            else (hash((self.req_id, time.time_ns())) & 0x7FFFFFFF)
        self.extra = {}
        if self.sampling.input_penalty and self.sampling.has_penalty:
            for t in shm_req.get_prompt_ids():
                self.out_token_counter[t] = self.out_token_counter.get(t, 0) + 1

    # ---- lengths ----
    def total_len(self) -> int:
        """Prompt + generated tokens (the last generated token has no KV yet)."""
        return self.shm_req.input_len + self.cur_output_len

    def need_prefill(self) -> bool:
        return self.cur_kv_len < self.total_len() - 1 or self.cur_output_len == 0

    def get_chunked_input_token_ids(self, chunk: int) -> np.ndarray:
        end = min(self.total_len(), self.cur_kv_len + chunk)
        return self.shm_req.shm_prompt_ids.arr[self.cur_kv_len:end]

    def get_last_gen_token(self) -> int:
        return int(self.shm_req.shm_prompt_ids.arr[self.total_len() - 1])

    # ---- output ----
    def append_token(self, token_id: int, logprob: float):
        r = self.shm_req
        idx = r.input_len + self.cur_output_len
        r.shm_prompt_ids.arr[idx] = token_id
        r.shm_logprobs.arr[idx] = logprob
        self.cur_output_len += 1
        self.cumlogprob += logprob
        if self.sampling.has_penalty:
            self.out_token_counter[token_id] = self.out_token_counter.get(token_id, 0) + 1

    def update_finish_status(self, eos_ids, max_total_len: Optional[int] = None):
        sp = self.sampling
        out_len = self.cur_output_len
        last = self.get_last_gen_token()
        if self.infer_aborted:
            self.finish_status.set_status(FinishStatus.FINISHED_ABORTED)
        elif self.stop_str_matched:
            self.finish_status.set_status(FinishStatus.FINISHED_STOP)
        elif out_len >= sp.min_new_tokens and self._stop_sequences_matched():
            self.finish_status.set_status(FinishStatus.FINISHED_STOP)
        elif out_len >= sp.min_new_tokens and not sp.ignore_eos and last in eos_ids:
            self.finish_status.set_status(FinishStatus.FINISHED_STOP)
        elif out_len >= sp.max_new_tokens:
            self.finish_status.set_status(FinishStatus.FINISHED_LENGTH)
        elif max_total_len is not None and self.total_len() >= max_total_len:
            self.finish_status.set_status(FinishStatus.FINISHED_LENGTH)

    def _stop_sequences_matched(self) -> bool:
        if not self.sampling.stop_sequences:
            return False
        r = self.shm_req
        out = r.shm_prompt_ids.arr[r.input_len: r.input_len + self.cur_output_len]
        for s in self.sampling.stop_sequences:
            n = len(s)
            if n <= out.shape[0] and out[-n:].tolist() == s:
                return True
        return False

    def publish(self):
        """Make this step's progress visible to the other processes.  Order matters: lengths and finish
        state first, `candetoken_out_len` last (the detokenizer reads everything below it)."""
        r = self.shm_req
        r.shm_cur_kv_len = self.cur_kv_len
        r.cumlogprob = self.cumlogprob
        r.shm_cur_output_len = self.cur_output_len
        if self.finish_status.is_finished():
            r.finish_token_index = r.input_len + self.cur_output_len - 1
            r.finish_status.set_status(self.finish_status.get_status())
        r.candetoken_out_len = self.cur_output_len


class InferenceContext:
    def __init__(self, model, radix_cache=None, vocab_size: Optional[int] = None):
        self.model = model
        self.req_manager = model.req_manager
        self.mem_manager = model.mem_manager
        self.radix_cache = radix_cache
        self.vocab_size = vocab_size or model.vocab
        self.requests: Dict[int, InferReq] = {}
        self.infer_req_ids: List[int] = []
        self.host_cache = None  # HostKVCache (second prefix-cache tier) when --enable_cpu_cache
        self.state_cache = None  # StateSnapshotCache of hybrid linear-attention models

    # ---- capacity ----
    def get_can_alloc_token_num(self) -> int:
        n = self.mem_manager.can_use_mem_size
        if self.radix_cache is not None:
            n += self.radix_cache.unreferenced_tokens_num()
        return n

    def alloc_slots(self, n: int) -> torch.Tensor:
        if self.radix_cache is not None:
            self.radix_cache.free_radix_cache_to_get_enough_token(n)
        return self.mem_manager.alloc(n)

    # ---- admission ----
    def add_req(self, shm_req: Req, dp_index: int = 0) -> Optional[InferReq]:
        idx = self.req_manager.alloc()
        if idx < 0:
            return None
        req = InferReq(shm_req, idx, self.vocab_size, dp_index)
        self.requests[req.req_id] = req
        self.infer_req_ids.append(req.req_id)
        self._match_radix_cache(req)
        return req

    def _match_radix_cache(self, req: InferReq):
        """Reuse cached KV of the longest known prefix of prompt[:-1] (the last prompt token must run
        through the model to produce the first output)."""
        if self.radix_cache is None or req.shm_req.sample_params.disable_prompt_cache or \
                req.shm_req.sample_params.prompt_logprobs >= 0:     # every prompt position must run through the model
            return
        ids = req.shm_req.shm_prompt_ids.arr[: max(req.total_len() - 1, 0)]
        node, n, slots = self.radix_cache.match_prefix(ids, update_refs=True)
        if self.state_cache is not None:
            # hybrid model: the match is only worth what the longest state snapshot inside it covers
            L, snap = (0, None) if node is None else self.state_cache.lookup(ids, n)
            if L == 0:
                if node is not None:
                    self.radix_cache.dec_node_ref_counter(node)
                return
            self.state_cache.restore(snap, req.req_idx, L)
            n, slots = L, slots[:L]
        if node is None:
            self._match_host_cache(req, ids, 0)
            return
        req.shared_kv_node = node
        req.shared_len = n
        req.cur_kv_len = n
        req.slots = slots.astype(np.int32)
        row = torch.from_numpy(req.slots)
        self.req_manager.req_to_token_indexs[req.req_idx, :n] = row.to(self.req_manager.device)
        if req.shm_req.prompt_cache_len == 0:
            req.shm_req.prompt_cache_len = n
        if self.state_cache is None:
            self._match_host_cache(req, ids, n)

    def _match_host_cache(self, req: InferReq, ids, n_gpu: int):
        """Extend the cached prefix with pages of the host tier: pages from the one containing token n_gpu on."""
        hc = self.host_cache
        if hc is None or len(ids) < hc.P:
            return
        from .host_kv_cache import page_keys

        keys = page_keys(ids, hc.P)
        p0 = n_gpu // hc.P
        m = hc.match(keys, p0)
        if m == 0 or (p0 + m) * hc.P <= n_gpu:
            return
        need = m * hc.P
        if self.get_can_alloc_token_num() < need + 64:
            return
        new = self.alloc_slots(need)
        hc.load(keys, p0, m, new)
        new_np = new.numpy().astype(np.int32)
        skip = n_gpu - p0 * hc.P          # tokens of the first page the GPU tree already covers
        if skip:
            self.mem_manager.free(new_np[:skip])
        use = new_np[skip:]
        end = (p0 + m) * hc.P
        req.slots = np.concatenate([req.slots[:n_gpu], use]) if n_gpu else use
        req.cur_kv_len = end
        self.req_manager.req_to_token_indexs[req.req_idx, n_gpu:end] = torch.from_numpy(use).to(self.req_manager.device)
        req.shm_req.cpu_prompt_cache_len = end - n_gpu
        if req.shm_req.prompt_cache_len < end:
            req.shm_req.prompt_cache_len = end

    # ---- release ----
    def free_a_req_mem(self, req: InferReq):
        """Donate the request's KV to the radix tree (or free it) and drop its tree reference."""
        n = req.cur_kv_len
        if self.host_cache is not None and n >= self.host_cache.P and not req.paused and \
                not req.shm_req.sample_params.disable_prompt_cache:
            self.host_cache.offload(req.shm_req.shm_prompt_ids.arr[:n], req.slots[:n])
        if self.radix_cache is None or req.shm_req.sample_params.disable_prompt_cache:
            own = req.slots[req.shared_len:n]
            if own.size:
                self.mem_manager.free(own)
        else:
            key = req.shm_req.shm_prompt_ids.arr[:n]
            present = self.radix_cache.insert(key, req.slots[:n])
            dup = req.slots[req.shared_len:present]  # positions the tree already had: our copies are spare
            if dup.size:
                self.mem_manager.free(dup)
        if req.shared_kv_node is not None:
            self.radix_cache.dec_node_ref_counter(req.shared_kv_node)
            req.shared_kv_node = None
        req.shared_len = 0
        req.cur_kv_len = 0
        req.slots = np.empty(0, dtype=np.int32)

    def remove_req(self, req: InferReq):
        self.free_a_req_mem(req)
        self.req_manager.free(req.req_idx)
        self.requests.pop(req.req_id, None)
        self.infer_req_ids.remove(req.req_id)
        req.shm_req.shm_infer_released = True

    # ---- memory pressure ----
    def pause_req(self, req: InferReq):
        """Give the KV back; the request re-prefills (usually from the radix tree) when recovered."""
        if req.paused:
            return
        self.free_a_req_mem(req)
        req.paused = True
        req.shm_req.is_paused = True

    def recover_req(self, req: InferReq):
        if not req.paused:
            return
        req.paused = False
        req.shm_req.is_paused = False
        self._match_radix_cache(req)
