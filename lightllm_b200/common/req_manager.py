"""Request slots: ``req_to_token_indexs[max_req + 1, max_seq_len]`` maps (request, position) to
a KV pool slot; row ``max_req`` is the HOLD request used to pad batches to a CUDA-graph size.
Also owns the per-request device arrays the sampler and the decode prologue read, so a decode
step's input ids never leave the GPU.

Behavioural counterpart: lightllm/common/req_manager.py.
"""
from __future__ import annotations

import torch


class ReqManager:
    def __init__(self, max_request_num: int, max_sequence_length: int, mem_manager, device: torch.device):
        self.max_request_num = max_request_num
        self.max_sequence_length = max_sequence_length
        self.HOLD_REQUEST_ID = max_request_num
        self.mem_manager = mem_manager
        self.device = device
        self.req_to_token_indexs = torch.zeros((max_request_num + 1, max_sequence_length), dtype=torch.int32,
                                               device=device)
        self.req_to_token_indexs[self.HOLD_REQUEST_ID].fill_(mem_manager.HOLD_TOKEN_MEMINDEX)
        # next input token of every request (written by the sampler, read by the decode prologue)
        self.req_to_next_token_ids = torch.zeros((max_request_num + 1, 8), dtype=torch.int64, device=device)
        # multimodal rotary: position of a decode token = sequence position + this offset (0 for text-only)
        self.req_to_position_delta = torch.zeros(max_request_num + 1, dtype=torch.int32, device=device)
        self._free = list(range(max_request_num - 1, -1, -1))

    @property
    def can_use_req_size(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            return -1
        return self._free.pop()

    def free(self, req_idx: int, free_token_index=None) -> None:
        self._free.append(req_idx)
        if free_token_index is not None and len(free_token_index) > 0:
            self.mem_manager.free(free_token_index)

    def free_all(self) -> None:
        self._free = list(range(self.max_request_num - 1, -1, -1))
