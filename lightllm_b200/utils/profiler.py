"""Per-process profiler control behind /profiler_start and /profiler_stop: torch profiler traces
(CPU + CUDA) written as TensorBoard traces under LIGHTLLM_TRACE_DIR, or one top-level NVTX range
for an external capture.  Reference: lightllm/utils/profiler.py:25-227.
"""
from __future__ import annotations

import os
import time


class ProcessProfiler:
    def __init__(self, mode: str, name: str):
        self.mode = mode
        self.name = name
        self.active = False
        self._prof = None
        self.trace_dir = os.environ.get("LIGHTLLM_TRACE_DIR", "./trace")

    def cmd(self, what: str):
        if what == "start":
            self.start()
        elif what == "stop":
            self.stop()
        else:
            raise ValueError(what)

    def start(self):
        if self.active:
            return
        self.active = True
        if self.mode == "torch_profiler":
            import torch

            os.makedirs(self.trace_dir, exist_ok=True)
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self._prof = torch.profiler.profile(
                activities=acts, record_shapes=True, with_stack=True,
                on_trace_ready=torch.profiler.tensorboard_trace_handler(self.trace_dir, worker_name=f"{self.name}_{int(time.time())}", use_gzip=True))
            self._prof.__enter__()
        elif self.mode == "nvtx":
            import torch

            if torch.cuda.is_available():
                torch.cuda.nvtx.range_push("LIGHTLLM_PROFILE")

    def stop(self):
        if not self.active:
            return
        self.active = False
        if self.mode == "torch_profiler" and self._prof is not None:
            self._prof.__exit__(None, None, None)
            self._prof = None
        elif self.mode == "nvtx":
            import torch

            if torch.cuda.is_available():
                torch.cuda.nvtx.range_pop()
