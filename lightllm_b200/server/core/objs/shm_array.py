"""Numpy arrays over POSIX shared memory (or process-local memory when `name` is None).

The HTTP worker creates the arrays of a request (token ids, logprobs); router, model ranks and
the detokenizer link to them by name.  Reference: lightllm/server/core/objs/shm_array.py and
lightllm/utils/shm_utils.py.
"""
from __future__ import annotations

import os
from multiprocessing import shared_memory
from typing import Optional

import numpy as np

from ....utils.shm_cleanup import get_cleanup, register_posix_shm_for_cleanup


def create_or_link_shm(name: str, size: int, force_create: bool = False, settle_s: float = 2.0):
    """Returns (SharedMemory, created).  Several processes of a server start side by side and may reach the same
    segment at the same moment: the one that loses the creation race waits until the winner has given the segment
    its size (a freshly created segment is empty for an instant) instead of judging it too small.  A segment that
    stays too small (left over from an earlier server with other limits) is replaced."""
    import time

    try:
        shm = shared_memory.SharedMemory(name=name, create=True, size=size)
        return shm, True
    except FileExistsError:
        t0 = time.time()
        while True:
            try:
                shm = shared_memory.SharedMemory(name=name, create=False)
            except FileNotFoundError:
                return create_or_link_shm(name, size, force_create, settle_s)    # it went away meanwhile: start over
            except ValueError:
                shm = None                        # still empty: cannot be mapped yet
            if shm is not None and shm.size >= size and not force_create:
                return shm, False
            if force_create or time.time() - t0 > settle_s:
                break
            if shm is not None:
                shm.close()
            time.sleep(0.01)
        if shm is not None:
            shm.close()
            try:
                shm.unlink()
            except FileNotFoundError:
                pass
        else:
            try:
                shared_memory.SharedMemory(name=name, create=False).unlink()
            except (FileNotFoundError, ValueError):
                try:
                    os.unlink("/dev/shm/" + name.lstrip("/"))
                except OSError:
                    pass
        shm = shared_memory.SharedMemory(name=name, create=True, size=size)
        return shm, True


def _untrack(shm):
    """Stop Python's resource tracker from unlinking a segment this process only linked to."""
    try:
        from multiprocessing import resource_tracker

        resource_tracker.unregister(shm._name, "shared_memory")
    except Exception:
        pass


class ShmArray:
    def __init__(self, name: Optional[str], shape, dtype):
        self.name = name
        self.shape = tuple(shape)
        self.dtype = np.dtype(dtype)
        self.shm = None
        self.arr = None
        self._owner = False

    @property
    def nbytes(self) -> int:
        return int(np.prod(self.shape)) * self.dtype.itemsize

    def create_shm(self):
        if self.name is None:
            self.arr = np.zeros(self.shape, dtype=self.dtype)
            return self
        self.shm, created = create_or_link_shm(self.name, max(self.nbytes, 1), force_create=True)
        self._owner = True
        register_posix_shm_for_cleanup(self.name)
        self.arr = np.ndarray(self.shape, dtype=self.dtype, buffer=self.shm.buf)
        return self

    def link_shm(self):
        if self.name is None:
            raise ValueError("a process-local array cannot be linked")
        self.shm = shared_memory.SharedMemory(name=self.name, create=False)
        self.arr = np.ndarray(self.shape, dtype=self.dtype, buffer=self.shm.buf)
        return self

    def close_shm(self, unlink: Optional[bool] = None):
        self.arr = None
        if self.shm is not None:
            self.shm.close()
            if unlink if unlink is not None else self._owner:
                try:
                    self.shm.unlink()
                except FileNotFoundError:
                    pass
                get_cleanup().unregister_posix(self.name)
            self.shm = None
