"""The request object shared by every process of a server.

`Req` is a fixed-layout ctypes structure: an array of them lives in one POSIX shared-memory
block, only slot indices travel over zmq.  Per-request side arrays (token ids of prompt +
output, logprobs) are separate shm arrays named after the slot.  The structure also works in
ordinary process memory (offline engine, tests).

Writers by field: the HTTP worker fills the request at admission and sets `is_aborted`; the
model rank (tp rank 0 of the replica) writes `shm_cur_kv_len`, `shm_cur_output_len`, the token
/ logprob arrays, `finish_status`, `finish_token_index`, then `candetoken_out_len` LAST (the
detokenizer trusts everything below that index); the detokenizer writes the text ring,
`stop_str_matched*` and `can_released_mark`.

Reference: lightllm/server/core/objs/req.py:24-546 (fields, FinishStatus, the token-budget
estimate of the past-future scheduler), out_token_circlequeue.py.
"""
from __future__ import annotations

import ctypes
import os
import time
from typing import List, Optional, Tuple

import numpy as np

from .sampling_params import MAX_PROMPT_LOGPROBS, SamplingParams
from .shm_array import ShmArray

LIGHTLLM_OUT_TOKEN_QUEUE_SIZE = int(os.getenv("LIGHTLLM_OUT_TOKEN_QUEUE_SIZE", 8))
LIGHTLLM_TOKEN_MAX_BYTES = int(os.getenv("LIGHTLLM_TOKEN_MAX_BYTES", 1280))
ADDED_OUTPUT_LEN = 16  # safety margin of the scheduler's output-length estimate
PREFIX_TOKEN_MAX = 4


class FinishStatus(ctypes.Structure):
    _pack_ = 4
    _fields_ = [("status", ctypes.c_int)]
    NO_FINISH, FINISHED_STOP, FINISHED_LENGTH, FINISHED_ABORTED, FINISHED_ERROR = 0, 1, 2, 3, 4
    _NAMES = {1: "stop", 2: "length", 3: "abort", 4: "error"}

    def __init__(self, status: int = 0):
        super().__init__()
        self.status = status

    def set_status(self, s: int):
        assert 0 <= s <= 4
        self.status = s

    def get_status(self) -> int:
        return self.status

    def is_finished(self) -> bool:
        return self.status != self.NO_FINISH

    def is_stopped(self) -> bool:
        return self.status == self.FINISHED_STOP

    def is_aborted(self) -> bool:
        return self.status == self.FINISHED_ABORTED

    def get_finish_reason(self) -> Optional[str]:
        return self._NAMES.get(self.status)


class TokenText(ctypes.Structure):
    """One decoded token as the detokenizer hands it to the HTTP worker: UTF-8 bytes (cut at
    LIGHTLLM_TOKEN_MAX_BYTES), the token's index in the request's id array, and what the stream needs with it."""

    _pack_ = 4
    _fields_ = [("data", ctypes.c_ubyte * LIGHTLLM_TOKEN_MAX_BYTES), ("data_len", ctypes.c_int),
                ("src_index", ctypes.c_int), ("special", ctypes.c_bool), ("count_output_tokens", ctypes.c_int)]

    def store(self, text: str, src_index: int, special: bool, count_output_tokens: int):
        raw = text.encode("utf-8")[:LIGHTLLM_TOKEN_MAX_BYTES]
        ctypes.memmove(self.data, raw, len(raw))
        self.data_len, self.src_index = len(raw), src_index
        self.special, self.count_output_tokens = special, count_output_tokens

    def load(self) -> Tuple[str, int, bool, int]:
        return (bytes(self.data[: self.data_len]).decode("utf-8", errors="replace"), self.src_index,
                bool(self.special), self.count_output_tokens)


class OutTokenRing(ctypes.Structure):
    """Decoded-token ring inside the shared request: one producer (the detokenizer process), one consumer (the
    HTTP worker).  `produced` and `consumed` are free-running counters (slot = counter mod size), each
    written by exactly one side, so all LIGHTLLM_OUT_TOKEN_QUEUE_SIZE slots can be in use and "empty" and "full"
    need no spare slot.  The producer fills the slot first and publishes by advancing `produced` afterwards.
    Reference: lightllm/server/core/objs/out_token_circlequeue.py (head / tail indices, one slot kept free)."""

    _pack_ = 4
    _fields_ = [("items", TokenText * LIGHTLLM_OUT_TOKEN_QUEUE_SIZE), ("consumed", ctypes.c_uint32),
                ("produced", ctypes.c_uint32)]
    CAPACITY = LIGHTLLM_OUT_TOKEN_QUEUE_SIZE
    WRAP = CAPACITY * ((1 << 31) // CAPACITY)   # counters wrap at a multiple of the size, whatever the size

    def reset(self):
        self.consumed = 0
        self.produced = 0

    def __len__(self) -> int:
        return (self.produced - self.consumed) % self.WRAP

    def is_empty(self) -> bool:
        return self.produced == self.consumed

    def is_full(self) -> bool:
        return len(self) >= self.CAPACITY

    # ---- producer ----
    def push(self, text: str, src_index: int, special: bool, count_output_tokens: int):
        if self.is_full():
            raise BufferError("out token ring is full")
        self.items[self.produced % self.CAPACITY].store(text, src_index, special, count_output_tokens)
        self.produced = (self.produced + 1) % self.WRAP

    # ---- consumer ----
    def peek(self) -> Tuple[str, int, bool, int]:
        if self.is_empty():
            raise BufferError("out token ring is empty")
        return self.items[self.consumed % self.CAPACITY].load()

    def pop_no_ret(self):
        if self.is_empty():
            raise BufferError("out token ring is empty")
        self.consumed = (self.consumed + 1) % self.WRAP

    def pop(self) -> Tuple[str, int, bool, int]:
        item = self.peek()
        self.pop_no_ret()
        return item


CircularQueue = OutTokenRing   # the reference's name for this structure


class PrefixTokenIds(ctypes.Structure):
    _pack_ = 4
    _fields_ = [("ids", ctypes.c_int * PREFIX_TOKEN_MAX), ("size", ctypes.c_int)]

    def set(self, ids):
        assert len(ids) <= PREFIX_TOKEN_MAX
        for i, v in enumerate(ids):
            self.ids[i] = v
        self.size = len(ids)

    def to_list(self):
        return list(self.ids[: self.size])


class Req(ctypes.Structure):
    _pack_ = 4
    _fields_ = [
        ("index_in_shm_mem", ctypes.c_int),
        ("ref_count", ctypes.c_int),
        ("recv_time", ctypes.c_double),
        ("request_id", ctypes.c_int64),
        ("group_req_id", ctypes.c_int64),
        ("input_len", ctypes.c_int),
        ("alloc_shm_numpy_len", ctypes.c_int),
        ("shm_infer_released", ctypes.c_bool),
        ("shm_cur_kv_len", ctypes.c_int),
        ("shm_cur_output_len", ctypes.c_int),
        ("candetoken_out_len", ctypes.c_int),
        ("prompt_cache_len", ctypes.c_int),
        ("cpu_prompt_cache_len", ctypes.c_int),
        ("disk_prompt_cache_len", ctypes.c_int),
        ("is_paused", ctypes.c_bool),
        ("finish_status", FinishStatus),
        ("is_aborted", ctypes.c_bool),
        ("finish_token_index", ctypes.c_int),
        ("out_tokens_queue", OutTokenRing),
        ("sample_params", SamplingParams),
        ("chunked_prefill_size", ctypes.c_int),
        ("router_max_wait_tokens", ctypes.c_int),
        ("prefix_token_ids", PrefixTokenIds),
        ("can_released_mark", ctypes.c_bool),
        ("reward_score", ctypes.c_float),
        ("cumlogprob", ctypes.c_float),
        ("mtp_accepted_token_num", ctypes.c_int),
        ("mtp_step", ctypes.c_int),
        ("stop_str_matched", ctypes.c_bool),
        ("stop_str_matched_token_index", ctypes.c_int),
        ("dp_index", ctypes.c_int),
        ("first_token_time", ctypes.c_double),
        ("routed_len", ctypes.c_int),          # tokens whose routed experts the rank wrote to the "routed" array
    ]

    # ---- life cycle ----
    def init(self, request_id: int, prompt_ids: List[int], sample_param, tokenizer=None, chunked_prefill_size: int = 0,
             router_max_wait_tokens: int = 1, mtp_step: int = 0, shm_prefix: Optional[str] = None,
             max_total_len: Optional[int] = None):
        """Fill a fresh request.  `shm_prefix` None keeps the side arrays process-local."""
        self.ref_count = max(self.ref_count, 0)
        self.recv_time = time.time()
        self.request_id = request_id
        self.group_req_id = int(sample_param.get("group_request_id", -1)) if isinstance(sample_param, dict) else -1
        self.is_paused = False
        self.finish_status = FinishStatus()
        self.is_aborted = False
        self.shm_infer_released = False
        self.shm_cur_kv_len = 0
        self.shm_cur_output_len = 0
        self.candetoken_out_len = 0
        self.prompt_cache_len = 0
        self.cpu_prompt_cache_len = 0
        self.disk_prompt_cache_len = 0
        self.finish_token_index = -1
        self.can_released_mark = False
        self.reward_score = float("nan")
        self.cumlogprob = 0.0
        self.mtp_accepted_token_num = 0
        self.mtp_step = mtp_step
        self.stop_str_matched = False
        self.stop_str_matched_token_index = -1
        self.dp_index = -1
        self.first_token_time = 0.0
        self.routed_len = 0
        self.out_tokens_queue.reset()
        if isinstance(sample_param, SamplingParams):
            ctypes.memmove(ctypes.byref(self.sample_params), ctypes.byref(sample_param), ctypes.sizeof(SamplingParams))
        else:
            self.sample_params.init(tokenizer, **(sample_param or {}))
        if self.group_req_id < 0:
            self.group_req_id = self.sample_params.group_request_id if self.sample_params.group_request_id >= 0 \
                else request_id
        self.prefix_token_ids.size = 0
        self.input_len = len(prompt_ids)
        total = self.input_len + self.sample_params.max_new_tokens
        if max_total_len is not None:
            total = min(total, max_total_len)
        self.alloc_shm_numpy_len = total + 8
        self.chunked_prefill_size = chunked_prefill_size if chunked_prefill_size > 0 else max(self.input_len, 1)
        self.router_max_wait_tokens = router_max_wait_tokens
        self._shm_prefix = shm_prefix
        self.create_prompt_ids_shm_array()
        self.create_logprobs_shm_array()
        self.shm_prompt_ids.arr[: self.input_len] = np.asarray(prompt_ids, dtype=np.int64)
        self.post_init()
        return self

    def post_init(self):
        pass

    def _name(self, kind: str) -> Optional[str]:
        prefix = getattr(self, "_shm_prefix", None)
        if prefix is None:
            return None
        return f"{prefix}_shm_{kind}_{self.index_in_shm_mem}"

    def create_prompt_ids_shm_array(self):
        self.shm_prompt_ids = ShmArray(self._name("prompts"), (self.alloc_shm_numpy_len,), np.int64).create_shm()

    def create_logprobs_shm_array(self):
        self.shm_logprobs = ShmArray(self._name("logprobs"), (self.alloc_shm_numpy_len,), np.float32).create_shm()

    PROMPT_TOPK_MAX = MAX_PROMPT_LOGPROBS

    def prompt_meta_cols(self) -> int:
        """Columns of the per-position prompt record: rank of the prompt token, then k ids and k logprobs of the
        k most likely tokens at that position (`prompt_logprobs` = k, capped)."""
        k = min(max(int(self.sample_params.prompt_logprobs), 0), self.PROMPT_TOPK_MAX)
        return 1 + 2 * k

    def create_prompt_meta_shm_array(self):
        self.shm_prompt_meta = ShmArray(self._name("pmeta"), (self.input_len + 1, self.prompt_meta_cols()),
                                        np.float32).create_shm()
        self.shm_prompt_meta.arr[:, 0] = -1.0

    def link_prompt_meta_shm_array(self, shm_prefix: str):
        self._shm_prefix = shm_prefix
        self.shm_prompt_meta = ShmArray(self._name("pmeta"), (self.input_len + 1, self.prompt_meta_cols()),
                                        np.float32).link_shm()

    def create_routed_shm_array(self, num_moe_layers: int, top_k: int, dtype):
        """Per-token routed expert ids [tokens, MoE layers, top_k], written by the model rank when the request
        finishes (`--enable_return_routed_experts`)."""
        self.shm_routed = ShmArray(self._name("routed"), (self.alloc_shm_numpy_len, num_moe_layers, top_k),
                                   dtype).create_shm()

    def link_routed_shm_array(self, shm_prefix: str, num_moe_layers: int, top_k: int, dtype):
        self._shm_prefix = shm_prefix
        self.shm_routed = ShmArray(self._name("routed"), (self.alloc_shm_numpy_len, num_moe_layers, top_k),
                                   dtype).link_shm()

    def link_prompt_ids_shm_array(self, shm_prefix: str):
        self._shm_prefix = shm_prefix
        self.shm_prompt_ids = ShmArray(self._name("prompts"), (self.alloc_shm_numpy_len,), np.int64).link_shm()

    def link_logprobs_shm_array(self, shm_prefix: str):
        self._shm_prefix = shm_prefix
        self.shm_logprobs = ShmArray(self._name("logprobs"), (self.alloc_shm_numpy_len,), np.float32).link_shm()

    def release_shm_arrays(self, unlink: bool = False):
        for a in ("shm_prompt_ids", "shm_logprobs", "shm_routed", "shm_prompt_meta"):
            arr = getattr(self, a, None)
            if arr is not None:
                arr.close_shm(unlink=unlink or None)
                setattr(self, a, None)

    # ---- views ----
    def get_prompt_ids(self) -> List[int]:
        return self.shm_prompt_ids.arr[: self.input_len].tolist()

    def get_prompt_ids_numpy(self) -> np.ndarray:
        return self.shm_prompt_ids.arr[: self.input_len]

    def get_output_ids(self) -> List[int]:
        return self.shm_prompt_ids.arr[self.input_len: self.input_len + self.shm_cur_output_len].tolist()

    def get_all_ids_numpy(self) -> np.ndarray:
        return self.shm_prompt_ids.arr[: self.input_len + self.shm_cur_output_len]

    def get_used_tokens(self) -> int:
        return max(0, self.shm_cur_kv_len)

    def get_str(self) -> str:
        return (f"request_id:{self.request_id}, input_len:{self.input_len}, shm_cur_kv_len:{self.shm_cur_kv_len}, "
                f"shm_cur_output_len:{self.shm_cur_output_len}, finished:{self.finish_status.is_finished()}")

    def can_release(self) -> bool:
        """The HTTP worker may recycle the slot: finished, drained, marked by the last stage, unreferenced."""
        if self.finish_status.is_finished() or self.stop_str_matched:
            return self.can_released_mark and self.ref_count == 1 and self.out_tokens_queue.is_empty()
        return False

    # ---- scheduler cost model (past-future estimate) ----
    def get_tuple_tokens(self, is_busy: bool, ema_req_out_len: int) -> Tuple[int, int]:
        """(a, b): a = KV tokens the request holds once its prompt is in, b = tokens it is still expected
        to grow by.  A busy router assumes every request runs to max_new_tokens; otherwise the estimate is
        max(1.1 x produced so far, moving average of finished lengths).  Chunked prefill keeps a request
        alive longer, which is modelled as extra output steps."""
        has_out = self.shm_cur_output_len
        sp = self.sample_params
        if sp.ignore_eos or is_busy:
            expect = sp.max_new_tokens
        else:
            expect = min(sp.max_new_tokens, max(int(1.1 * has_out), ema_req_out_len))
        a_len = max(self.input_len + has_out + 1, self.shm_cur_kv_len + 1)
        remaining_prefill = self.input_len + has_out - self.shm_cur_kv_len
        chunks = (remaining_prefill + self.chunked_prefill_size - 1) // self.chunked_prefill_size
        b_len = chunks * (self.router_max_wait_tokens + 1) + expect - has_out - 1
        return a_len, max(0, b_len) + ADDED_OUTPUT_LEN

    def get_decode_need_tokens(self) -> int:
        need = min(self.input_len + self.shm_cur_output_len - self.shm_cur_kv_len, self.chunked_prefill_size)
        if need == 1 and self.mtp_step > 0:
            need = (self.mtp_step + 1) * 2
        return need

    def get_first_router_need_tokens(self) -> int:
        return min(self.input_len + self.shm_cur_output_len, self.chunked_prefill_size)


class TokenHealingReq(Req):
    """Token healing: the last (up to 2) prompt tokens are regenerated under a prefix constraint."""

    _pack_ = 4

    def post_init(self):
        for n in (2, 1):
            if self.input_len > n:
                ids = self.shm_prompt_ids.arr[self.input_len - n: self.input_len].tolist()
                self.input_len -= n
                self.prefix_token_ids.set(ids)
                # room for the regenerated tokens
                self.sample_params.max_new_tokens += n + 6
                return
