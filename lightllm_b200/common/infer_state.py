"""Per-forward data carried between the engine and the model.

`ModelInput` is what the engine hands to `model.forward` (reference:
lightllm/common/basemodel/batch_objs.py); `InferState` is the per-forward scratch every layer
reads (reference: lightllm/common/basemodel/infer_struct.py).  Index tensors are int32 on the
model's device; in a step they are written once by the step-prologue kernel.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch


@dataclass
class ModelInput:
    batch_size: int
    total_token_num: int                 # sum of kv lengths after this step (for scheduling stats)
    max_kv_len: int                      # longest sequence (incl. new tokens) in the batch
    is_prefill: bool
    b_req_idx: torch.Tensor              # int32 [B]
    b_seq_len: torch.Tensor              # int32 [B]  kv length after this step
    mem_indexes: torch.Tensor            # int32 [T]  pool slot of every new token
    input_ids: Optional[torch.Tensor] = None       # int64 [T] (prefill; decode reads req_to_next_token_ids)
    b_ready_cache_len: Optional[torch.Tensor] = None  # int32 [B] (prefill) tokens already in the pool
    b_q_len: Optional[torch.Tensor] = None         # int32 [B] (prefill) new tokens per request
    max_q_len: int = 1
    b_prefill_has_output: Optional[List[bool]] = None  # chunked prefill: does this chunk end the prompt
    multimodal_params: Optional[list] = None
    return_all_logits: bool = False      # prompt_logprobs: logits for every prompt position
    b_mtp_index: Optional[torch.Tensor] = None
    return_hidden: bool = False          # speculative decoding: also return the final residual stream [T, hidden]
    draft_input_hidden: Optional[torch.Tensor] = None  # draft modules: hidden state of the target model per token
    verify_pass: bool = False            # speculative decoding: a pass whose later positions may be rolled back


@dataclass
class ModelOutput:
    logits: torch.Tensor                 # fp32 [B or T, vocab]
    hidden: Optional[torch.Tensor] = None


@dataclass
class InferState:
    is_prefill: bool
    batch_size: int
    num_tokens: int
    max_kv_len: int
    max_q_len: int
    b_req_idx: torch.Tensor
    b_seq_len: torch.Tensor
    mem_index: torch.Tensor
    position_ids: torch.Tensor = None            # rotary position of every token (families may remap it)
    seq_pos: torch.Tensor = None                 # index of every token inside its request (causal limit)
    cu_q: Optional[torch.Tensor] = None           # int32 [B+1]
    b_ready_cache_len: Optional[torch.Tensor] = None
    batch_of_token: Optional[torch.Tensor] = None
    decode_num_splits: int = 1
    decode_scratch: Optional[tuple] = None
    extra: dict = field(default_factory=dict)
