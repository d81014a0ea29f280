"""Incremental detokenisation with two offsets.

For each request keep `prefix_offset` and `read_offset` into its output ids: decode the windows
[prefix:read] and [prefix:] and emit the suffix only if the longer text grew and does not end in
U+FFFD (an incomplete multi-byte character).  Reference: lightllm/server/detokenization/decode.py:7-35.
"""
from __future__ import annotations

from typing import List


class DecodeReq:
    def __init__(self, req, is_pd_decode_mode: bool = False):
        self.req = req
        self.request_id = req.request_id
        self.group_req_id = req.group_req_id
        self.input_len = req.input_len
        self.prefix_str = ""
        self.output_ids: List[int] = []
        self.output_strs: List[str] = []
        self.prefix_offset = 0
        self.read_offset = 0
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
    ids = decode_req.output_ids
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
