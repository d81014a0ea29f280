"""Symmetric device memory: the same-sized region on every rank, mapped into all peers of the node
through CUDA IPC, so that kernels can load from / store to a peer's memory over NVLink.

`SymmetricRegion(nbytes, pstate)` allocates the local block (cudaMalloc, zeroed), exchanges IPC handles
over the host-side process group and opens the peers' blocks.  `ptrs[q]` is the base address of rank
q's block as seen from this rank; `tensor(offset, shape, dtype)` is a zero-copy torch view of the local
block (so a GEMM can write its output straight into memory the peers can read).
"""
from __future__ import annotations

import ctypes
from typing import List

import torch
import torch.distributed as dist

from ..ops._native import check, kernels

_DT = {torch.bfloat16: ("<V2", 2), torch.float32: ("<f4", 4), torch.int32: ("<i4", 4), torch.uint8: ("|u1", 1),
       torch.float16: ("<f2", 2)}


class _RawCuda:
    """Exposes a raw device range through the CUDA array interface so torch can view it without owning it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def view_device_memory(ptr: int, nbytes: int, device) -> torch.Tensor:
    return torch.as_tensor(_RawCuda(ptr, nbytes), device=device)


class SymmetricRegion:
    def __init__(self, nbytes: int, rank: int, world: int, group=None, device=None, local_only: bool = False):
        self.nbytes = int(nbytes)
        self.rank, self.world = rank, world
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        lib = kernels()
        p = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            check(lib.llb_symm_alloc(ctypes.byref(p), ctypes.c_int64(self.nbytes)), "symm_alloc")
        self.local_ptr = p.value
        self.ptrs: List[int] = [0] * world
        self.ptrs[rank] = self.local_ptr
        self._opened = []
        self._bytes = view_device_memory(self.local_ptr, self.nbytes, self.device)
        if world > 1 and not local_only:
            handle = (ctypes.c_ubyte * 64)()
            check(lib.llb_ipc_get_handle(ctypes.c_void_p(self.local_ptr), handle), "ipc_get_handle")
            all_handles = [None] * world
            dist.all_gather_object(all_handles, bytes(handle), group=group)
            for q, h in enumerate(all_handles):
                if q == rank:
                    continue
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                out = ctypes.c_void_p()
                check(lib.llb_ipc_open_handle(buf, ctypes.byref(out)), "ipc_open_handle")
                self.ptrs[q] = out.value
                self._opened.append(out.value)

    def tensor(self, offset: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * _DT[dtype][1]
        assert offset % 16 == 0 and offset + nbytes <= self.nbytes
        return self._bytes[offset:offset + nbytes].view(dtype).view(*shape)

    def close(self):
        lib = kernels()
        for p in self._opened:
            lib.llb_ipc_close_handle(ctypes.c_void_p(p))
        self._opened = []
        if self.local_ptr:
            self._bytes = None
            lib.llb_symm_free(ctypes.c_void_p(self.local_ptr))
            self.local_ptr = 0
