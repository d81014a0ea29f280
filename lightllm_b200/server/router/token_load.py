"""Per-replica load figures in shared memory, read by /token_load and by the PD master's
adaptive-load selector: [current usage, estimated peak usage ("logical"), dynamic max load].
Reference: lightllm/server/router/token_load.py.
"""
from __future__ import annotations

from ..core.objs.atomic_lock import SharedArray


class TokenLoad:
    def __init__(self, name: str, dp_size_in_node: int = 1):
        self.dp = dp_size_in_node
        self.arr = SharedArray(name, (dp_size_in_node, 3), "float64")

    def set(self, dp_index: int, current: float, logical: float, dynamic: float):
        self.arr.arr[dp_index, 0] = current
        self.arr.arr[dp_index, 1] = logical
        self.arr.arr[dp_index, 2] = dynamic

    def get_current_load(self, dp_index: int = 0) -> float:
        return float(self.arr.arr[dp_index, 0])

    def get_logical_max_load(self, dp_index: int = 0) -> float:
        return float(self.arr.arr[dp_index, 1])

    def get_dynamic_max_load(self, dp_index: int = 0) -> float:
        return float(self.arr.arr[dp_index, 2])

    def snapshot(self):
        return [{"current_load": self.get_current_load(i), "logical_max_load": self.get_logical_max_load(i),
                 "dynamic_max_load": self.get_dynamic_max_load(i)} for i in range(self.dp)]
