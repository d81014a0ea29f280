"""Sub-allocator that hands out tensor views of one pre-allocated byte workspace.

Used where a step needs scratch tensors of changing shapes without touching the caching allocator (CUDA-graph
capture, communication staging): `alloc(shape, dtype)` returns a view into the workspace at an aligned offset,
`free(tensor)` gives the range back; adjacent free ranges are merged, the smallest fitting free range is taken.

Reference: lightllm/utils/tensor_buffer_manager.py.
"""
from __future__ import annotations

import bisect
from typing import Dict, List, Sequence, Tuple, Union

import torch

Shape = Union[int, Sequence[int], torch.Size]


class TensorBufferManager:
    def __init__(self, buffer: torch.Tensor, alignment_bytes: int = 256):
        assert buffer.dim() == 1 and buffer.dtype == torch.uint8 and buffer.is_contiguous(), \
            "the workspace is a flat uint8 tensor"
        assert alignment_bytes > 0 and alignment_bytes & (alignment_bytes - 1) == 0
        self.buffer = buffer
        self.align = alignment_bytes
        base = buffer.data_ptr() if buffer.numel() else 0
        self._skew = (-base) % alignment_bytes       # first aligned byte of the workspace
        self.capacity = max(buffer.numel() - self._skew, 0) // alignment_bytes * alignment_bytes
        self._free: List[Tuple[int, int]] = [(0, self.capacity)] if self.capacity else []   # sorted (offset, size)
        self._live: Dict[int, Tuple[int, int]] = {}  # data_ptr -> (offset, size)

    def _up(self, n: int) -> int:
        return (n + self.align - 1) // self.align * self.align

    @property
    def free_bytes(self) -> int:
        return sum(s for _, s in self._free)

    @property
    def largest_free_block(self) -> int:
        return max((s for _, s in self._free), default=0)

    def alloc(self, shape: Shape, dtype: torch.dtype) -> torch.Tensor:
        shape = torch.Size((shape,) if isinstance(shape, int) else tuple(shape))
        if shape.numel() == 0:
            return torch.empty(shape, dtype=dtype, device=self.buffer.device)
        esize = torch.empty((), dtype=dtype).element_size()
        need = self._up(max(shape.numel() * esize, 1))
        best = -1
        for i, (_, size) in enumerate(self._free):
            if size >= need and (best < 0 or size < self._free[best][1]):
                best = i
        if best < 0:
            raise MemoryError(f"workspace exhausted: want {need} bytes, largest free block {self.largest_free_block}")
        off, size = self._free.pop(best)
        if size > need:
            self._free.insert(best, (off + need, size - need))
        start = self._skew + off
        t = self.buffer[start:start + shape.numel() * esize].view(dtype).view(shape)
        self._live[self.buffer.data_ptr() + start] = (off, need)
        return t

    def free(self, tensor: torch.Tensor) -> None:
        if tensor.numel() == 0:
            return
        rec = self._live.pop(tensor.data_ptr(), None)
        if rec is None:
            raise ValueError("tensor was not allocated from this workspace (or was freed already)")
        off, size = rec
        i = bisect.bisect_left(self._free, (off, 0))
        self._free.insert(i, (off, size))
        # merge with the right, then the left neighbour
        if i + 1 < len(self._free) and self._free[i][0] + self._free[i][1] == self._free[i + 1][0]:
            self._free[i] = (off, self._free[i][1] + self._free.pop(i + 1)[1])
        if i > 0 and self._free[i - 1][0] + self._free[i - 1][1] == self._free[i][0]:
            o, s = self._free[i - 1]
            self._free[i - 1] = (o, s + self._free.pop(i)[1])

    def reset(self):
        self._free = [(0, self.capacity)] if self.capacity else []
        self._live.clear()
