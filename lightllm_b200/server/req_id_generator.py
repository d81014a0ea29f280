"""Request ids: a group id advances by MAX_BEST_OF (8); sub-request i of a group is group_id + i.
The counter lives in shared memory so several HTTP workers hand out disjoint ids.
Reference: lightllm/server/req_id_generator.py.
"""
from __future__ import annotations

from .core.objs.atomic_lock import SharedInt
from .core.objs.sampling_params import MAX_BEST_OF
from .core.objs.start_args import get_unique_server_name


class ReqIDGenerator:
    def __init__(self, name: str = None, start: int = 0):
        self._counter = SharedInt(f"{name or get_unique_server_name()}_req_id_gen")
        if self._counter.get_value() < start:
            self._counter.set_value(start)

    def generate_id(self) -> int:
        return self._counter.add(MAX_BEST_OF)


def convert_sub_id_to_group_id(sub_req_id: int) -> int:
    return (sub_req_id // MAX_BEST_OF) * MAX_BEST_OF
