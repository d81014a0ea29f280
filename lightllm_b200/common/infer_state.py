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


class ShardedLogits:
    """Vocabulary-parallel logits: this rank holds columns [v0, v0 + local.shape[1]) of the [rows, vocab] matrix.

    With tensor parallelism the lm_head is split over the vocabulary.  Gathering the full fp32 matrix on every
    rank costs rows x vocab x 4 bytes of all-gather per step (131 MB at batch 256 for a 128k vocabulary); a greedy
    step only needs each shard's (max, arg-max, sum of exponentials) per row, a few KB.  `greedy()` does that;
    `full()` is the gather for everything that needs the whole row (random sampling, penalties, token masks,
    prompt logprobs).  Reference: lightllm/models/llama/layer_infer/post_layer_infer.py:88-117 always gathers.
    """

    def __init__(self, local: torch.Tensor, tp, v0: int, vocab: int):
        self.local, self.tp, self.v0, self.vocab = local, tp, int(v0), int(vocab)
        self._full = None

    @property
    def shape(self):
        return (self.local.shape[0], self.vocab)

    @property
    def device(self):
        return self.local.device

    def __getitem__(self, rows):
        assert not isinstance(rows, tuple), "only rows of vocabulary-parallel logits can be selected"
        return ShardedLogits(self.local[rows], self.tp, self.v0, self.vocab)

    def index_select(self, dim, index):
        assert dim == 0
        return ShardedLogits(self.local.index_select(0, index), self.tp, self.v0, self.vocab)

    def full(self) -> torch.Tensor:
        if self._full is None:
            self._full = self.tp.gather_logits(self.local)
        return self._full

    def greedy(self):
        """(ids int64 [rows], logprob fp32 [rows]) of the arg-max token, identical on every rank."""
        import torch.distributed as dist

        from .. import ops

        part = ops.greedy_partials(self.local, self.v0)
        B = part.shape[0]
        parts = torch.empty((self.tp.size * B, *part.shape[1:]), dtype=part.dtype, device=part.device)
        dist.all_gather_into_tensor(parts, part, group=self.tp.group)
        return ops.greedy_merge(parts.view(self.tp.size, B, *part.shape[1:]))


class ModelOutput:
    """`logits_any`: fp32 [B or T, vocab] tensor, or ShardedLogits when the lm_head is vocabulary-parallel (hand
    it to `ops.sample`); `logits`: always the dense matrix; `hidden`: final residual stream when asked for."""

    def __init__(self, logits=None, hidden: Optional[torch.Tensor] = None):
        self.logits_any, self.hidden = logits, hidden

    @property
    def logits(self) -> torch.Tensor:
        """The dense [rows, vocab] matrix (gathered on first use when the model produced vocabulary shards)."""
        x = self.logits_any
        return x.full() if isinstance(x, ShardedLogits) else x


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
