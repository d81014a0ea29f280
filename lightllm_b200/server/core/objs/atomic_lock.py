"""Cross-process locks and counters on words in POSIX shared memory, backed by the C++ atomics
of the runtime library (`std::atomic` compare-exchange on the mapped word).

Reference: lightllm/server/core/objs/atomic_lock.py, atomic_array_lock.py and
router/dynamic_prompt/shared_arr.py (which use the `atomics` cffi package).
"""
from __future__ import annotations

import asyncio
import ctypes
import time

import numpy as np

from ....ops._native import runtime
from .shm_array import create_or_link_shm


def _lib():
    lib = runtime()
    if not getattr(lib, "_atomic_typed", False):
        vp = ctypes.c_void_p
        lib.llb_atomic_load_i32.argtypes = [vp]
        lib.llb_atomic_load_i32.restype = ctypes.c_int32
        lib.llb_atomic_store_i32.argtypes = [vp, ctypes.c_int32]
        lib.llb_atomic_add_i32.argtypes = [vp, ctypes.c_int32]
        lib.llb_atomic_add_i32.restype = ctypes.c_int32
        lib.llb_atomic_cas_i32.argtypes = [vp, ctypes.c_int32, ctypes.c_int32]
        lib.llb_atomic_cas_i32.restype = ctypes.c_int32
        lib.llb_atomic_load_i64.argtypes = [vp]
        lib.llb_atomic_load_i64.restype = ctypes.c_int64
        lib.llb_atomic_store_i64.argtypes = [vp, ctypes.c_int64]
        lib.llb_atomic_add_i64.argtypes = [vp, ctypes.c_int64]
        lib.llb_atomic_add_i64.restype = ctypes.c_int64
        lib.llb_spin_lock.argtypes = [vp, ctypes.c_int64]
        lib.llb_spin_lock.restype = ctypes.c_int32
        lib.llb_spin_unlock.argtypes = [vp]
        lib._atomic_typed = True
    return lib


def _addr(buf, offset=0) -> int:
    return ctypes.addressof(ctypes.c_char.from_buffer(buf, offset))


class LockTimeout(TimeoutError):
    pass


class AtomicShmLock:
    """One spin lock in its own 4-byte shm segment.  `with lock:` acquires (bounded wait)."""

    def __init__(self, lock_name: str, timeout_s: float = 30.0):
        self.lock_name = lock_name
        self.timeout_ns = int(timeout_s * 1e9)
        self.shm, created = create_or_link_shm(lock_name, 8)
        self._p = _addr(self.shm.buf)
        self._lib = _lib()
        if created:
            self._lib.llb_atomic_store_i32(self._p, 0)

    def acquire(self):
        if not self._lib.llb_spin_lock(self._p, self.timeout_ns):
            raise LockTimeout(f"lock {self.lock_name} not acquired in time (holder died?)")

    def release(self):
        self._lib.llb_spin_unlock(self._p)

    def __enter__(self):
        self.acquire()
        return self

    def __exit__(self, *exc):
        self.release()
        return False

    def force_release(self):
        """Recovery hook for a supervisor that knows the holder is dead."""
        self._lib.llb_spin_unlock(self._p)


class AtomicLockItem:
    def __init__(self, lib, p, timeout_ns):
        self._lib, self._p, self._t = lib, p, timeout_ns

    def __enter__(self):
        if not self._lib.llb_spin_lock(self._p, self._t):
            raise LockTimeout("array lock not acquired in time")
        return self

    def __exit__(self, *exc):
        self._lib.llb_spin_unlock(self._p)
        return False


class AtomicShmArrayLock:
    """`lock_num` independent spin locks in one shm segment (one per request slot)."""

    def __init__(self, lock_name: str, lock_num: int, timeout_s: float = 30.0):
        self.lock_num = lock_num
        self.shm, created = create_or_link_shm(lock_name, 4 * lock_num)
        self._base = _addr(self.shm.buf)
        self._lib = _lib()
        self._t = int(timeout_s * 1e9)
        if created:
            for i in range(lock_num):
                self._lib.llb_atomic_store_i32(self._base + 4 * i, 0)

    def get_lock_context(self, index: int) -> AtomicLockItem:
        assert 0 <= index < self.lock_num
        return AtomicLockItem(self._lib, self._base + 4 * index, self._t)


class AsyncLock:
    """asyncio-friendly wrapper: polls the shm lock without blocking the event loop."""

    def __init__(self, lock: AtomicShmLock):
        self.lock = lock

    async def __aenter__(self):
        lib, p = self.lock._lib, self.lock._p
        t0 = time.time()
        while not lib.llb_atomic_cas_i32(p, 0, 1):
            await asyncio.sleep(0)
            if time.time() - t0 > self.lock.timeout_ns / 1e9:
                raise LockTimeout(self.lock.lock_name)
        return self

    async def __aexit__(self, *exc):
        self.lock.release()
        return False


class SharedInt:
    """int64 in shared memory with atomic load / store / add."""

    def __init__(self, name: str, init=None):
        self.name = name
        self.shm, created = create_or_link_shm(name, 8)
        self._p = _addr(self.shm.buf)
        self._lib = _lib()
        if created:
            self._lib.llb_atomic_store_i64(self._p, 0 if init is None else init)
        elif init is not None:
            self._lib.llb_atomic_store_i64(self._p, init)

    def set_value(self, v: int):
        self._lib.llb_atomic_store_i64(self._p, int(v))

    def get_value(self) -> int:
        return int(self._lib.llb_atomic_load_i64(self._p))

    def add(self, v: int = 1) -> int:
        """Returns the value before the addition."""
        return int(self._lib.llb_atomic_add_i64(self._p, int(v)))


class SharedArray:
    """Plain numpy array in shared memory (single writer per element by convention)."""

    def __init__(self, name: str, shape, dtype):
        self.shape = tuple(shape)
        self.dtype = np.dtype(dtype)
        size = int(np.prod(self.shape)) * self.dtype.itemsize
        self.shm, created = create_or_link_shm(name, max(size, 8))
        self.arr = np.ndarray(self.shape, dtype=self.dtype, buffer=self.shm.buf)
        if created:
            self.arr[...] = 0
