"""Health monitor process: polls /health and, after consecutive failures, kills the whole server
process tree so that an external supervisor (k8s, systemd) restarts it.  There is no in-process recovery
of a failed rank: recovery = restart.  Reference: lightllm/server/health_monitor/manager.py:18-49.
"""
from __future__ import annotations

import os
import time

import requests

from ...utils.process_utils import kill_tree, set_proc_title, start_parent_check_thread
from ..core.objs.start_args import StartArgs

CHECK_INTERVAL_S = float(os.getenv("HEALTH_CHECK_INTERVAL_SECONDS", 88))
FAILURE_THRESHOLD = int(os.getenv("HEALTH_CHECK_FAILURE_THRESHOLD", 3))


class HealthMonitor:
    def __init__(self, args: StartArgs, get=requests.get, kill=kill_tree, sleep=time.sleep):
        self.url = f"http://127.0.0.1:{args.port}/health"
        self.failures = 0
        self._get, self._kill, self._sleep = get, kill, sleep
        self.parent = os.getppid()

    def check_once(self) -> bool:
        try:
            ok = self._get(self.url, timeout=60).status_code == 200
        except Exception:
            ok = False
        self.failures = 0 if ok else self.failures + 1
        return ok

    def run(self, max_iters=None):
        n = 0
        while max_iters is None or n < max_iters:
            n += 1
            self._sleep(CHECK_INTERVAL_S)
            self.check_once()
            if self.failures >= FAILURE_THRESHOLD:
                self._kill(self.parent)
                return "killed"
        return "stopped"


def start_health_check_process(args_dict: dict, pipe_writer):
    args = StartArgs.from_dict(args_dict)
    set_proc_title(f"lightllm::{args.unique_server_name}::health_monitor")
    start_parent_check_thread()
    mon = HealthMonitor(args)
    pipe_writer.send("init ok")
    mon.run()
