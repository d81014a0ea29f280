"""Process helpers: titles, parent-death watchdog, graceful shutdown, child supervision.
Reference: lightllm/utils/process_check.py, graceful_utils.py, start_utils.py.
"""
from __future__ import annotations

import multiprocessing as mp
import os
import signal
import sys
import threading
import time
from typing import Callable, List, Optional

import psutil


def set_proc_title(title: str):
    try:
        import setproctitle

        setproctitle.setproctitle(title)
    except Exception:
        pass


def start_parent_check_thread(interval_s: float = 2.0):
    """Children exit when their parent is gone (the launcher owns the process tree)."""
    parent = os.getppid()

    def watch():
        while True:
            if os.getppid() != parent or not psutil.pid_exists(parent):
                os._exit(1)
            time.sleep(interval_s)

    t = threading.Thread(target=watch, daemon=True)
    t.start()
    return t


def graceful_registry(name: str):
    def handler(signum, frame):
        sys.exit(0)

    try:
        signal.signal(signal.SIGTERM, handler)
    except ValueError:
        pass  # not in the main thread


def kill_tree(pid: int, include_self: bool = True):
    try:
        p = psutil.Process(pid)
    except psutil.NoSuchProcess:
        return
    for c in p.children(recursive=True):
        try:
            c.kill()
        except psutil.NoSuchProcess:
            pass
    if include_self:
        try:
            p.kill()
        except psutil.NoSuchProcess:
            pass


class SubmoduleManager:
    """Starts sub-processes and waits for each one's "init ok" over a pipe; supervises them afterwards:
    if any child exits, everything is torn down (recovery = restart the server)."""

    def __init__(self):
        self.processes: List[mp.Process] = []
        self.ctx = mp.get_context("spawn")

    def start_submodule_processes(self, start_funcs: List[Callable], start_args: List[tuple], timeout_s: float = 3600):
        pipes, procs = [], []
        for fn, a in zip(start_funcs, start_args):
            r, w = self.ctx.Pipe(duplex=False)
            p = self.ctx.Process(target=fn, args=(*a, w), daemon=False)
            p.start()
            pipes.append(r)
            procs.append(p)
        def give_up():
            # the processes of this call are not registered yet: they go down with the registered ones, or the
            # launcher would wait for them for ever when it exits
            for q in procs:
                if q.is_alive():
                    kill_tree(q.pid)
            self.terminate_all()

        for p, r, fn in zip(procs, pipes, start_funcs):
            t0 = time.time()
            while not r.poll(0.2):
                if not p.is_alive():
                    give_up()
                    raise RuntimeError(f"{fn.__name__} died during start-up (exit code {p.exitcode})")
                if time.time() - t0 > timeout_s:
                    give_up()
                    raise TimeoutError(f"{fn.__name__} start-up timed out")
            msg = r.recv()
            if msg != "init ok":
                give_up()
                raise RuntimeError(f"{fn.__name__} failed to start: {msg}")
        self.processes.extend(procs)
        return procs

    def terminate_all(self):
        for p in self.processes:
            if p.is_alive():
                kill_tree(p.pid)
        self.processes = []

    def any_dead(self) -> Optional[mp.Process]:
        for p in self.processes:
            if not p.is_alive():
                return p
        return None

    def supervise(self, extra_alive_checks: Optional[List[Callable[[], bool]]] = None, interval_s: float = 1.0):
        """Blocks until a child dies or a check fails, then tears everything down."""
        while True:
            dead = self.any_dead()
            if dead is not None:
                break
            if extra_alive_checks and not all(c() for c in extra_alive_checks):
                break
            time.sleep(interval_s)
        self.terminate_all()


process_manager = SubmoduleManager()
