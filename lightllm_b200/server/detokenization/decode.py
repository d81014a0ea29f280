"""Incremental detokenisation with two offsets.

For each request keep `prefix_offset` and `read_offset` into its output ids: decode the windows
[prefix:read] and [prefix:] and emit the suffix only if the longer text grew and does not end in
U+FFFD (an incomplete multi-byte character).  The window starts inside the prompt: its last
`LIGHTLLM_DECODE_PREFIX_LENGTH` (default 5) tokens are decoded along as context, so that tokenizers which write a
word's leading space only after another token (SentencePiece-style) give the first generated word its space.
Reference: lightllm/server/detokenization/decode.py:7-35, decode_req.py:9-30.
"""
from __future__ import annotations

import os
from typing import List


def prompt_context_len() -> int:
    try:
        return max(0, int(os.environ.get("LLB_DECODE_PREFIX_LENGTH", os.environ.get("LIGHTLLM_DECODE_PREFIX_LENGTH", "5"))))
    except ValueError:
        return 5


class DecodeReq:
    def __init__(self, req, is_pd_decode_mode: bool = False):
        self.req = req
        self.request_id = req.request_id
        self.group_req_id = req.group_req_id
        self.input_len = req.input_len
        self.prefix_str = ""
        self.output_ids: List[int] = []
        self.output_strs: List[str] = []
        # the end of the prompt, as far back as it holds real token ids (a picture's virtual ids are not text)
        tail: List[int] = []
        k = prompt_context_len()
        arr = getattr(getattr(req, "shm_prompt_ids", None), "arr", None)
        if k > 0 and arr is not None and self.input_len > 0:
            tail = [int(t) for t in arr[max(0, self.input_len - k):self.input_len]]
        self.prompt_tail = tail
        self.context_ids: List[int] = list(tail)      # prompt tail + output ids: what the windows index into
        self._tail_checked = False
        self.prefix_offset = 0
        self.read_offset = len(tail)
        self.stop_strs = req.sample_params.stop_sequences.to_strings()
        self.stop_tail_len = max((len(s) for s in self.stop_strs), default=0) + 16
        sp = req.sample_params
        self.skip_special_tokens = sp.skip_special_tokens
        self.add_spaces_between_special_tokens = sp.add_spaces_between_special_tokens
        self.print_eos_token = sp.print_eos_token
        self.out_queue_is_full_count = 0

    def need_detoken(self) -> bool:
        return (not self.req.is_aborted or True) and len(self.output_ids) < self.req.candetoken_out_len

    def out_queue_is_full(self) -> bool:
        return self.req.out_tokens_queue.is_full()

    def get_next_token_id_and_index(self):
        src_index = self.input_len + len(self.output_ids)
        return int(self.req.shm_prompt_ids.arr[src_index]), src_index

    def get_decode_tokens(self):
        return self.prefix_offset, self.read_offset

    def stop_sequences_str_match(self) -> bool:
        if not self.stop_strs:
            return False
        tail = "".join(self.output_strs[-self.stop_tail_len:])
        return any(s in tail for s in self.stop_strs)

    def can_set_release_mark(self) -> bool:
        r = self.req
        if r.is_aborted:
            return True
        if r.stop_str_matched:
            return True
        return r.finish_status.is_finished() and r.candetoken_out_len == len(self.output_ids) \
            and r.finish_token_index == self.input_len + len(self.output_ids) - 1


def decode_token(tokenizer, decode_req: DecodeReq, new_token_id: int, eos_ids) -> str:
    """Returns the new text produced by appending `new_token_id` (possibly empty)."""
    decode_req.output_ids.append(new_token_id)
    if new_token_id in eos_ids and not decode_req.print_eos_token:
        decode_req.output_strs.append("")
        return ""
    if not decode_req._tail_checked:      # first token: drop prompt context that is not in the vocabulary
        decode_req._tail_checked = True
        try:
            vocab = len(tokenizer)
        except TypeError:
            vocab = None
        tail = decode_req.prompt_tail
        if vocab is not None:
            bad = [i for i, t in enumerate(tail) if t < 0 or t >= vocab]
            if bad:
                tail = tail[bad[-1] + 1:]
        decode_req.context_ids = list(tail)
        decode_req.prefix_offset, decode_req.read_offset = 0, len(tail)
    decode_req.context_ids.append(new_token_id)
    ids = decode_req.context_ids
    kw = dict(skip_special_tokens=decode_req.skip_special_tokens)
    prefix_text = tokenizer.decode(ids[decode_req.prefix_offset:decode_req.read_offset], **kw)
    new_text = tokenizer.decode(ids[decode_req.prefix_offset:], **kw)
    if len(new_text) > len(prefix_text) and not new_text.endswith("�"):
        out = new_text[len(prefix_text):]
        decode_req.prefix_offset = decode_req.read_offset
        decode_req.read_offset = len(ids)
    else:
        out = ""
    decode_req.output_strs.append(out)
    return out
