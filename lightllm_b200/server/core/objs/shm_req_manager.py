"""The shm array of `Req` structures and its slot management.

One POSIX shm block holds `running_max_req_size` requests; a free list (also in shm, guarded
by a cross-process spin lock) hands out slots; `ref_count` tracks how many processes currently
hold a Python view of a slot.  Reference: lightllm/server/core/objs/shm_req_manager.py:18-191.
"""
from __future__ import annotations

import ctypes
from typing import Type

import numpy as np

from .atomic_lock import AtomicShmArrayLock, AtomicShmLock
from .req import Req, TokenHealingReq
from .shm_array import create_or_link_shm
from .start_args import get_env_start_args, get_unique_server_name


class ShmReqManager:
    def __init__(self, server_name: str = None, max_req_num: int = None, req_class: Type[Req] = None):
        args = get_env_start_args()
        self.server_name = server_name or get_unique_server_name()
        self.max_req_num = max_req_num or args.running_max_req_size
        self.req_class = req_class or (TokenHealingReq if args.token_healing_mode else Req)
        self.req_size = ctypes.sizeof(self.req_class)
        self.shm, created = create_or_link_shm(f"{self.server_name}_req_shm_total", self.req_size * self.max_req_num)
        self.reqs = (self.req_class * self.max_req_num).from_buffer(self.shm.buf)
        # free list: int32[max_req_num + 1]; [0] = count, [1..count] = free slot ids
        self.free_shm, fl_created = create_or_link_shm(f"{self.server_name}_req_free_list", 4 * (self.max_req_num + 1))
        self.free = np.ndarray((self.max_req_num + 1,), dtype=np.int32, buffer=self.free_shm.buf)
        self.alloc_lock = AtomicShmLock(f"{self.server_name}_req_alloc_lock")
        self.slot_locks = AtomicShmArrayLock(f"{self.server_name}_req_slot_locks", self.max_req_num)
        if created or fl_created:
            with self.alloc_lock:
                for i in range(self.max_req_num):
                    self.reqs[i].ref_count = 0
                    self.reqs[i].index_in_shm_mem = i
                self.free[0] = self.max_req_num
                self.free[1:] = np.arange(self.max_req_num - 1, -1, -1, dtype=np.int32)

    def get_req_class_type(self):
        return self.req_class

    def free_count(self) -> int:
        return int(self.free[0])

    def alloc_req_index(self):
        with self.alloc_lock:
            n = int(self.free[0])
            if n == 0:
                return None
            idx = int(self.free[n])
            self.free[0] = n - 1
        return idx

    async def async_alloc_req_index(self):
        return self.alloc_req_index()

    def release_req_index(self, req_index: int):
        assert self.reqs[req_index].ref_count == 0, "slot released while still referenced"
        with self.alloc_lock:
            n = int(self.free[0])
            self.free[n + 1] = req_index
            self.free[0] = n + 1

    def get_req_obj_by_index(self, req_index: int) -> Req:
        with self.slot_locks.get_lock_context(req_index):
            r = self.reqs[req_index]
            r.ref_count += 1
        return r

    def put_back_req_obj(self, req: Req):
        idx = req.index_in_shm_mem
        with self.slot_locks.get_lock_context(idx):
            req.ref_count -= 1
            left = req.ref_count
        return left

    async def async_get_req_obj_by_index(self, req_index: int) -> Req:
        return self.get_req_obj_by_index(req_index)

    async def async_put_back_req_obj(self, req: Req):
        left = self.put_back_req_obj(req)
        if left == 0:
            req.release_shm_arrays(unlink=True)
        return left

    async def async_release_req_index(self, req_index: int):
        self.release_req_index(req_index)

    def close(self, unlink: bool = False):
        self.reqs = None
        self.free = None
        for shm in (self.shm, self.free_shm):
            try:
                shm.close()
                if unlink:
                    shm.unlink()
            except Exception:
                pass
