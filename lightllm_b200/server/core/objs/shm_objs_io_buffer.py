"""Router -> model-rank mailbox in shared memory.

Layout: int32[0] = readers that still have to consume the current message, int32[1] = pickle
length, int64 at byte 8 = generation counter, payload from byte 16.  The router writes only when
the reader count is 0, then publishes by setting the count to the number of local ranks and
bumping the generation; each rank polls the generation (no collective in the polling loop),
unpickles, and decrements the count.  Reference: lightllm/server/core/objs/shm_objs_io_buffer.py.
"""
from __future__ import annotations

import ctypes
import pickle
from typing import Any

from .atomic_lock import _addr, _lib
from .shm_array import create_or_link_shm

DEFAULT_BYTES = int(64 * 1024 * 1024)


class ShmObjsIOBuffer:
    HEADER = 16

    def __init__(self, name: str, node_world_size: int, size: int = DEFAULT_BYTES):
        self.name = name
        self.node_world_size = node_world_size
        self.shm, created = create_or_link_shm(name, size)
        self.size = self.shm.size
        self._lib = _lib()
        self._p = _addr(self.shm.buf)
        if created:
            self._lib.llb_atomic_store_i32(self._p, 0)
            self._lib.llb_atomic_store_i32(self._p + 4, 0)
            self._lib.llb_atomic_store_i64(self._p + 8, 0)

    # ---- writer (router) ----
    def is_empty(self) -> bool:
        return self._lib.llb_atomic_load_i32(self._p) == 0

    def write_obj(self, obj: Any):
        data = pickle.dumps(obj)
        if len(data) > self.size - self.HEADER:
            raise ValueError(f"mailbox message of {len(data)} bytes exceeds the {self.size}-byte buffer")
        self.shm.buf[self.HEADER:self.HEADER + len(data)] = data
        self._lib.llb_atomic_store_i32(self._p + 4, len(data))

    def set_ready(self):
        self._lib.llb_atomic_store_i32(self._p, self.node_world_size)
        self._lib.llb_atomic_add_i64(self._p + 8, 1)

    # ---- readers (ranks) ----
    def generation(self) -> int:
        return int(self._lib.llb_atomic_load_i64(self._p + 8))

    def is_ready(self) -> bool:
        return self._lib.llb_atomic_load_i32(self._p) > 0

    def read_obj(self) -> Any:
        n = self._lib.llb_atomic_load_i32(self._p + 4)
        return pickle.loads(bytes(self.shm.buf[self.HEADER:self.HEADER + n]))

    def sub_state(self):
        prev = self._lib.llb_atomic_add_i32(self._p, -1)
        assert prev > 0, "mailbox consumed more often than published"
