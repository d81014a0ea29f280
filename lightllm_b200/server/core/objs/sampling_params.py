"""Fixed-layout sampling parameters that live inside a shared-memory request.

A ctypes structure (no pointers) so that the HTTP worker can write it into POSIX shared memory
and the router / model ranks / detokenizer read the same bytes.  Field set, defaults and
validation follow the reference's public contract
(lightllm/server/core/objs/sampling_params.py:323-456): `do_sample=False` means greedy
(top_k forced to 1), `temperature < 1e-5` means greedy, at most 10 stop sequences of 256 tokens.
"""
from __future__ import annotations

import ctypes
import json
import os
from typing import List, Optional, Union

MAX_STOP_SEQUENCES = int(os.getenv("LIGHTLLM_MAX_STOP_SEQUENCES", 10))
STOP_SEQUENCE_MAX_LENGTH = int(os.getenv("LIGHTLLM_STOP_SEQUENCE_MAX_LENGTH", 256))
STOP_STR_MAX_BYTES = int(os.getenv("LIGHTLLM_STOP_SEQUENCE_STR_MAX_LENGTH", 256))
ALLOWED_TOKEN_IDS_MAX = int(os.getenv("LIGHTLLM_ALLOWED_TOKEN_IDS_MAX_LENGTH", 256))
INVALID_TOKEN_IDS_MAX = int(os.getenv("LIGHTLLM_INVALID_TOKEN_IDS_MAX_LENGTH", 10))
CONSTRAINT_MAX_BYTES = int(os.getenv("LIGHTLLM_REGULAR_CONSTRAINT_MAX_LENGTH", 2048))
GRAMMAR_MAX_BYTES = int(os.getenv("LIGHTLLM_GRAMMAR_CONSTRAINT_MAX_LENGTH", 2048))
JSON_SCHEMA_MAX_BYTES = int(os.getenv("LIGHTLLM_JSON_SCHEMA_MAX_LENGTH", 2048))
MAX_BEST_OF = 8
INPUT_PENALTY_DEFAULT = os.getenv("INPUT_PENALTY", "False").upper() in ("ON", "TRUE", "1")
# most alternatives per prompt position that `prompt_logprobs` may ask for (they are kept in shared memory per request)
MAX_PROMPT_LOGPROBS = int(os.getenv("LIGHTLLM_MAX_PROMPT_LOGPROBS", 20))
# default of `skip_special_tokens` for requests that do not say (the OpenAI routes set it themselves)
SKIP_SPECIAL_TOKENS = os.getenv("SKIP_SPECIAL_TOKENS", "False").upper() in ("ON", "TRUE", "1")


class ParamError(ValueError):
    """Invalid request parameter (HTTP 400)."""


class _Bytes(ctypes.Structure):
    """UTF-8 text in a fixed buffer."""

    CAP = 0

    def set(self, text: Optional[str]):
        data = (text or "").encode("utf-8")
        if len(data) > self.CAP:
            raise ParamError(f"text longer than {self.CAP} bytes")
        ctypes.memmove(self.buf, data, len(data))
        self.length = len(data)

    def get(self) -> str:
        return bytes(self.buf[: self.length]).decode("utf-8")


def _bytes_type(name, cap):
    return type(name, (_Bytes,), {"_pack_": 4, "_fields_": [("buf", ctypes.c_ubyte * cap), ("length", ctypes.c_int)],
                                  "CAP": cap})


RegularConstraint = _bytes_type("RegularConstraint", CONSTRAINT_MAX_BYTES)
GuidedGrammar = _bytes_type("GuidedGrammar", GRAMMAR_MAX_BYTES)
GuidedJsonSchema = _bytes_type("GuidedJsonSchema", JSON_SCHEMA_MAX_BYTES)


class _IntList(ctypes.Structure):
    CAP = 0

    def set(self, ids):
        ids = list(ids or [])
        if len(ids) > self.CAP:
            raise ParamError(f"too many token ids ({len(ids)} > {self.CAP})")
        for i, v in enumerate(ids):
            self.ids[i] = int(v)
        self.size = len(ids)

    def to_list(self) -> List[int]:
        return list(self.ids[: self.size])


def _intlist_type(name, cap):
    return type(name, (_IntList,), {"_pack_": 4, "_fields_": [("ids", ctypes.c_int * cap), ("size", ctypes.c_int)],
                                    "CAP": cap})


AllowedTokenIds = _intlist_type("AllowedTokenIds", ALLOWED_TOKEN_IDS_MAX)
InvalidTokenIds = _intlist_type("InvalidTokenIds", INVALID_TOKEN_IDS_MAX)


class StopSequence(ctypes.Structure):
    _pack_ = 4
    _fields_ = [("sequence", ctypes.c_int * STOP_SEQUENCE_MAX_LENGTH), ("size", ctypes.c_int),
                ("text", ctypes.c_ubyte * STOP_STR_MAX_BYTES), ("text_len", ctypes.c_int)]

    def set(self, ids: List[int], text: str = ""):
        if len(ids) > STOP_SEQUENCE_MAX_LENGTH:
            raise ParamError("stop sequence too long")
        for i, v in enumerate(ids):
            self.sequence[i] = int(v)
        self.size = len(ids)
        data = text.encode("utf-8")[:STOP_STR_MAX_BYTES]
        ctypes.memmove(self.text, data, len(data))
        self.text_len = len(data)

    def ids(self) -> List[int]:
        return list(self.sequence[: self.size])

    def string(self) -> str:
        return bytes(self.text[: self.text_len]).decode("utf-8", errors="ignore")


class StopSequenceGroups(ctypes.Structure):
    _pack_ = 4
    _fields_ = [("groups", StopSequence * MAX_STOP_SEQUENCES), ("size", ctypes.c_int)]

    def set(self, stop, tokenizer):
        """stop: None | str | List[str] | List[List[int]]."""
        if stop is None:
            self.size = 0
            return
        if isinstance(stop, str):
            stop = [stop]
        if len(stop) > MAX_STOP_SEQUENCES:
            raise ParamError(f"at most {MAX_STOP_SEQUENCES} stop sequences")
        for i, s in enumerate(stop):
            if isinstance(s, str):
                ids = tokenizer.encode(s, add_special_tokens=False) if tokenizer is not None else []
                self.groups[i].set(ids, s)
            else:
                self.groups[i].set(list(s), "")
        self.size = len(stop)

    def to_list(self) -> List[List[int]]:
        return [self.groups[i].ids() for i in range(self.size)]

    def to_strings(self) -> List[str]:
        out = [self.groups[i].string() for i in range(self.size)]
        return [s for s in out if s]


class ExponentialDecayLengthPenalty(ctypes.Structure):
    _pack_ = 4
    _fields_ = [("item0", ctypes.c_int), ("item1", ctypes.c_float)]

    def set(self, v):
        v = v or (1, 1.0)
        if not (isinstance(v, (list, tuple)) and len(v) == 2 and int(v[0]) >= 0 and float(v[1]) >= 1.0):
            raise ParamError("exponential_decay_length_penalty must be (start_index >= 0, factor >= 1.0)")
        self.item0, self.item1 = int(v[0]), float(v[1])

    def to_tuple(self):
        return (self.item0, self.item1)


class NodeUUId(ctypes.Structure):
    _pack_ = 4
    _fields_ = [("high", ctypes.c_uint64), ("low", ctypes.c_uint64)]

    def set(self, node_id: int):
        self.high = (node_id >> 64) & 0xFFFFFFFFFFFFFFFF
        self.low = node_id & 0xFFFFFFFFFFFFFFFF

    def get(self) -> int:
        return (self.high << 64) | self.low


class PDKVTransParams(ctypes.Structure):
    """What a decode node needs to receive this request's KV from its prefill node."""

    _pack_ = 4
    _fields_ = [("prefill_node_id", NodeUUId), ("decode_node_id", NodeUUId), ("peer_ip", ctypes.c_ubyte * 64),
                ("peer_ip_len", ctypes.c_int), ("peer_port", ctypes.c_int), ("master_req_id", ctypes.c_int64),
                ("valid", ctypes.c_bool), ("decode_dp", ctypes.c_int), ("decode_tp", ctypes.c_int)]

    def set(self, d: Optional[dict]):
        self.valid = bool(d)
        if not d:
            return
        self.prefill_node_id.set(int(d.get("prefill_node_id", 0)))
        self.decode_node_id.set(int(d.get("decode_node_id", 0)))
        ip = str(d.get("peer_ip", "")).encode()[:64]
        ctypes.memmove(self.peer_ip, ip, len(ip))
        self.peer_ip_len = len(ip)
        self.peer_port = int(d.get("peer_port", 0))
        self.master_req_id = int(d.get("master_req_id", 0))
        self.decode_dp = int(d.get("decode_dp", 1) or 1)      # replicas and ranks of the decode node: the KV of a
        self.decode_tp = int(d.get("decode_tp", 1) or 1)      # request goes to the replica that will serve it

    def to_dict(self):
        if not self.valid:
            return None
        return {"prefill_node_id": self.prefill_node_id.get(), "decode_node_id": self.decode_node_id.get(),
                "peer_ip": bytes(self.peer_ip[: self.peer_ip_len]).decode(), "peer_port": self.peer_port,
                "master_req_id": self.master_req_id, "decode_dp": max(1, self.decode_dp),
                "decode_tp": max(1, self.decode_tp)}


class SamplingParams(ctypes.Structure):
    _pack_ = 4
    _fields_ = [
        ("best_of", ctypes.c_int),
        ("n", ctypes.c_int),
        ("do_sample", ctypes.c_bool),
        ("presence_penalty", ctypes.c_float),
        ("frequency_penalty", ctypes.c_float),
        ("repetition_penalty", ctypes.c_float),
        ("temperature", ctypes.c_float),
        ("top_p", ctypes.c_float),
        ("top_k", ctypes.c_int),
        ("ignore_eos", ctypes.c_bool),
        ("image_max_patch_num", ctypes.c_int),
        ("max_new_tokens", ctypes.c_int),
        ("min_new_tokens", ctypes.c_int),
        ("input_penalty", ctypes.c_bool),
        ("regular_constraint", RegularConstraint),
        ("guided_grammar", GuidedGrammar),
        ("guided_json", GuidedJsonSchema),
        ("allowed_token_ids", AllowedTokenIds),
        ("invalid_token_ids", InvalidTokenIds),
        ("stop_sequences", StopSequenceGroups),
        ("exponential_decay_length_penalty", ExponentialDecayLengthPenalty),
        ("group_request_id", ctypes.c_int64),
        ("suggested_dp_index", ctypes.c_int),
        ("pd_master_node_id", NodeUUId),
        ("pd_kv_trans_params", PDKVTransParams),
        ("skip_special_tokens", ctypes.c_bool),
        ("add_special_tokens", ctypes.c_bool),
        ("add_spaces_between_special_tokens", ctypes.c_bool),
        ("print_eos_token", ctypes.c_bool),
        ("disable_prompt_cache", ctypes.c_bool),
        ("seed", ctypes.c_int64),
        ("prompt_logprobs", ctypes.c_int),
    ]

    # class-level defaults, overridable from the model's generation_config.json
    _defaults = {"do_sample": False, "presence_penalty": 0.0, "frequency_penalty": 0.0, "repetition_penalty": 1.0,
                 "temperature": 1.0, "top_p": 1.0, "top_k": -1}

    @classmethod
    def load_generation_cfg(cls, model_dir: str):
        """Defaults from generation_config.json (reference: sampling_params.py:403-420)."""
        path = os.path.join(model_dir or "", "generation_config.json")
        if not os.path.exists(path):
            return
        try:
            with open(path) as f:
                g = json.load(f)
            for k in list(cls._defaults):
                if k in g and g[k] is not None:
                    cls._defaults[k] = g[k]
        except Exception:
            pass

    def init(self, tokenizer=None, **kw):
        d = SamplingParams._defaults
        self.best_of = int(kw.get("best_of", 1))
        self.n = int(kw.get("n", self.best_of))
        self.do_sample = bool(kw.get("do_sample", d["do_sample"]))
        self.presence_penalty = float(kw.get("presence_penalty", d["presence_penalty"]))
        self.frequency_penalty = float(kw.get("frequency_penalty", d["frequency_penalty"]))
        self.repetition_penalty = float(kw.get("repetition_penalty", d["repetition_penalty"]))
        self.temperature = float(kw.get("temperature", d["temperature"]))
        self.top_p = float(kw.get("top_p", d["top_p"]))
        self.top_k = int(kw.get("top_k", d["top_k"]))
        self.ignore_eos = bool(kw.get("ignore_eos", False))
        self.image_max_patch_num = int(kw.get("image_max_patch_num", -1))
        self.max_new_tokens = int(kw.get("max_new_tokens", 65535))
        self.min_new_tokens = int(kw.get("min_new_tokens", 1))
        self.input_penalty = bool(kw.get("input_penalty", INPUT_PENALTY_DEFAULT))
        self.regular_constraint.set(kw.get("regular_constraint"))
        self.guided_grammar.set(kw.get("guided_grammar"))
        gj = kw.get("guided_json")
        self.guided_json.set(json.dumps(gj) if isinstance(gj, (dict, list)) else gj)
        self.allowed_token_ids.set(kw.get("allowed_token_ids"))
        lb = kw.get("logit_bias")
        invalid = kw.get("invalid_token_ids") or ([int(k) for k in lb.keys()] if isinstance(lb, dict) else None)
        self.invalid_token_ids.set(invalid)
        self.stop_sequences.set(kw.get("stop_sequences"), tokenizer)
        self.exponential_decay_length_penalty.set(kw.get("exponential_decay_length_penalty"))
        self.group_request_id = int(kw.get("group_request_id", -1))
        self.suggested_dp_index = int(kw.get("suggested_dp_index", -1))
        self.pd_master_node_id.set(int(kw.get("pd_master_node_id", 0)))
        self.pd_kv_trans_params.set(kw.get("pd_kv_trans_params"))
        self.skip_special_tokens = bool(kw.get("skip_special_tokens", SKIP_SPECIAL_TOKENS))
        self.add_special_tokens = bool(kw.get("add_special_tokens", True))
        self.add_spaces_between_special_tokens = bool(kw.get("add_spaces_between_special_tokens", True))
        self.print_eos_token = bool(kw.get("print_eos_token", False))
        self.disable_prompt_cache = bool(kw.get("disable_prompt_cache", False))
        seed = kw.get("seed", -1)
        self.seed = -1 if seed is None else int(seed)
        pl = kw.get("prompt_logprobs", -1)
        self.prompt_logprobs = -1 if pl is None else int(pl)
        if self.prompt_logprobs < -1 or self.prompt_logprobs > MAX_PROMPT_LOGPROBS:
            raise ValueError(f"prompt_logprobs must be in [-1, {MAX_PROMPT_LOGPROBS}], got {self.prompt_logprobs}")
        if not self.do_sample:  # greedy
            self.temperature, self.top_p, self.top_k = 1.0, 1.0, 1
        elif self.temperature < 1e-5:
            self.top_k = 1
        return self

    def verify(self, vocab_size: Optional[int] = None):
        if self.best_of <= 0 or self.best_of > MAX_BEST_OF:
            raise ParamError(f"best_of must be in [1, {MAX_BEST_OF}], got {self.best_of}")
        if self.n != self.best_of:
            raise ParamError("n must equal best_of")
        if self.n > 1 and not self.do_sample:
            raise ParamError("n > 1 needs do_sample=true")
        if self.presence_penalty < 0.0:
            raise ParamError("presence_penalty must be non-negative")
        if self.frequency_penalty < 0.0:
            raise ParamError("frequency_penalty must be non-negative")
        if self.repetition_penalty < 1.0:
            raise ParamError("repetition_penalty must be >= 1.0")
        if self.temperature < 0.0:
            raise ParamError("temperature must be non-negative")
        if not (0.0 < self.top_p <= 1.0):
            raise ParamError("top_p must be in (0, 1]")
        if self.top_k < -1 or self.top_k == 0:
            raise ParamError("top_k must be -1 (disabled) or >= 1")
        if self.max_new_tokens < 1:
            raise ParamError("max_new_tokens must be at least 1")
        if self.min_new_tokens < 1 or self.min_new_tokens > self.max_new_tokens:
            raise ParamError("min_new_tokens must be in [1, max_new_tokens]")
        n_constraints = sum(1 for c in (self.regular_constraint, self.guided_grammar, self.guided_json)
                            if c.length > 0)
        if n_constraints > 1:
            raise ParamError("only one of regular_constraint / guided_grammar / guided_json may be set")
        if vocab_size is not None:
            for t in self.allowed_token_ids.to_list() + self.invalid_token_ids.to_list():
                if t < 0 or t >= vocab_size:
                    raise ParamError(f"token id {t} out of vocabulary")
        return self

    @property
    def is_greedy(self) -> bool:
        return self.top_k == 1

    def to_dict(self) -> dict:
        return {"best_of": self.best_of, "n": self.n, "do_sample": self.do_sample,
                "presence_penalty": self.presence_penalty, "frequency_penalty": self.frequency_penalty,
                "repetition_penalty": self.repetition_penalty, "temperature": self.temperature, "top_p": self.top_p,
                "top_k": self.top_k, "ignore_eos": self.ignore_eos, "max_new_tokens": self.max_new_tokens,
                "min_new_tokens": self.min_new_tokens, "input_penalty": self.input_penalty,
                "stop_sequences": self.stop_sequences.to_list(), "seed": self.seed,
                "skip_special_tokens": self.skip_special_tokens, "add_special_tokens": self.add_special_tokens,
                "print_eos_token": self.print_eos_token, "disable_prompt_cache": self.disable_prompt_cache,
                "prompt_logprobs": self.prompt_logprobs,
                "regular_constraint": self.regular_constraint.get(), "guided_grammar": self.guided_grammar.get(),
                "guided_json": self.guided_json.get(), "allowed_token_ids": self.allowed_token_ids.to_list(),
                "invalid_token_ids": self.invalid_token_ids.to_list(),
                "exponential_decay_length_penalty": self.exponential_decay_length_penalty.to_tuple(),
                "group_request_id": self.group_request_id, "suggested_dp_index": self.suggested_dp_index}
