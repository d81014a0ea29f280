"""Removal of this process's shared-memory segments when it ends, however it ends.

Segments created by a server process (request arrays, the embedding arena, the shm request pool) are registered
here by name; at interpreter exit, or on SIGINT / SIGTERM / SIGHUP, every registered POSIX segment is unlinked (signal handlers are installed on request: `get_cleanup(signals=True)`) and
every registered System-V segment is marked for removal.  Only the creating process registers a segment; processes
that link to it do not.

`check_shm_size(args)` compares the size of /dev/shm with what the configured request pool, embedding arena and
host KV tier need and returns (available GiB, recommended GiB, ok).

Reference: lightllm/utils/auto_shm_cleanup.py, lightllm/utils/shm_size_check.py.
"""
from __future__ import annotations

import atexit
import ctypes
import ctypes.util
import logging
import os
import re
import signal
import threading
from typing import Dict, Optional, Set, Tuple

log = logging.getLogger(__name__)

IPC_RMID = 0


class ShmCleanup:
    def __init__(self, install_signal_handlers: bool = False):
        self._posix: Set[str] = set()
        self._sysv: Dict[int, Optional[int]] = {}
        self._lock = threading.Lock()
        self._pid = os.getpid()
        self._libc = None
        self._prev = {}
        atexit.register(self.cleanup)
        if install_signal_handlers:
            self.install_signal_handlers()

    def install_signal_handlers(self):
        """SIGINT / SIGTERM / SIGHUP run the cleanup first and then what was installed before (main thread only)."""
        if self._prev or threading.current_thread() is not threading.main_thread():
            return
        for sig in (signal.SIGINT, signal.SIGTERM, signal.SIGHUP):
            try:
                self._prev[sig] = signal.signal(sig, self._on_signal)
            except (ValueError, OSError):
                pass

    def _c(self):
        if self._libc is None:
            self._libc = ctypes.CDLL(ctypes.util.find_library("c") or "libc.so.6", use_errno=True)
        return self._libc

    def register_posix(self, name: str):
        with self._lock:
            self._posix.add(name.lstrip("/"))

    def unregister_posix(self, name: str):
        with self._lock:
            self._posix.discard(name.lstrip("/"))

    def register_sysv(self, key: int, shmid: Optional[int] = None):
        with self._lock:
            self._sysv[int(key)] = shmid

    def _on_signal(self, signum, frame):
        self.cleanup()
        prev = self._prev.get(signum)
        if callable(prev):
            prev(signum, frame)
        elif prev == signal.SIG_DFL or prev is None:
            signal.signal(signum, signal.SIG_DFL)
            os.kill(os.getpid(), signum)

    def cleanup(self):
        if os.getpid() != self._pid:  # a forked child inherits the registry but owns nothing
            return
        with self._lock:
            posix, sysv = list(self._posix), dict(self._sysv)
            self._posix.clear()
            self._sysv.clear()
        for name in posix:
            try:
                os.unlink(os.path.join("/dev/shm", name))
            except FileNotFoundError:
                pass
            except OSError as e:
                log.warning("could not unlink shared memory %s: %s", name, e)
        for key, shmid in sysv.items():
            try:
                libc = self._c()
                if shmid is None:
                    shmid = libc.shmget(ctypes.c_int(key), ctypes.c_size_t(0), ctypes.c_int(0))
                if shmid is not None and shmid >= 0:
                    libc.shmctl(ctypes.c_int(shmid), ctypes.c_int(IPC_RMID), None)
            except Exception as e:  # noqa: BLE001
                log.warning("could not remove System-V segment %#x: %s", key, e)


_INSTANCE: Optional[ShmCleanup] = None


def get_cleanup(signals: bool = False) -> ShmCleanup:
    """The process's registry (exit hook always; signal handlers when some caller asked for them)."""
    global _INSTANCE
    if _INSTANCE is None or _INSTANCE._pid != os.getpid():
        _INSTANCE = ShmCleanup()
    if signals:
        _INSTANCE.install_signal_handlers()
    return _INSTANCE


def register_posix_shm_for_cleanup(name: str):
    get_cleanup().register_posix(name)


def register_sysv_shm_for_cleanup(key: int, shmid: Optional[int] = None):
    get_cleanup().register_sysv(key, shmid)


# ------------------------------------------------------------------ /dev/shm size
def system_shm_gib(path: str = "/dev/shm") -> float:
    try:
        st = os.statvfs(path)
        return st.f_frsize * st.f_blocks / 2 ** 30
    except OSError:
        return 0.0


def recommended_shm_gib(args, max_image_pixels: int = 3940 * 2160, dtype_size: int = 2) -> float:
    """Request pool (token id + logprob arrays of every running request), the embedding arena, raw multimodal
    payloads of the cached items and the host KV tier when it lives in shared memory."""
    g = lambda k, d: getattr(args, k, None) or d  # noqa: E731
    reqs = int(g("running_max_req_size", 1000))
    max_len = int(g("max_req_total_len", 16384))
    req_pool = reqs * max_len * (8 + 4) * 1.25
    total = req_pool
    if getattr(args, "enable_multimodal", False):
        cap = int(g("cache_capacity", 200))
        total += cap * max_image_pixels * 3                                   # raw payloads
        total += int(g("embed_cache_storage_size", 4)) * 2 ** 30              # embedding arena (GiB flag)
    if getattr(args, "enable_cpu_cache", False):
        total += float(g("cpu_cache_storage_size", 2)) * 2 ** 30
    return total / 2 ** 30


def check_shm_size(args, path: str = "/dev/shm") -> Tuple[float, float, bool]:
    have, want = system_shm_gib(path), recommended_shm_gib(args)
    ok = have >= want
    if not ok:
        log.warning("%s has %.1f GiB, the configuration wants about %.1f GiB (docker: --shm-size)", path, have, want)
    return have, want, ok


# ------------------------------------------------------------------ segments of servers that were killed
_SERVER_SEGMENT = re.compile(r"^(llb(\d+)x[0-9a-f]{6})_")


def orphan_segments(path: str = "/dev/shm", pid_alive=None) -> dict:
    """Segments named after a launcher (`llb<launcher pid>x<tag>_...`) whose launcher no longer runs and that
    belong to this user: {server name: [file names]}.  A server that is killed outright (SIGKILL, out of memory)
    cannot remove its segments; everything else removes them on the way out."""
    if pid_alive is None:
        def pid_alive(pid: int) -> bool:
            try:
                os.kill(pid, 0)
                return True
            except ProcessLookupError:
                return False
            except PermissionError:
                return True
    out: dict = {}
    try:
        names = os.listdir(path)
    except OSError:
        return out
    for n in names:
        m = _SERVER_SEGMENT.match(n)
        if m is None or pid_alive(int(m.group(2))):
            continue
        try:
            if os.stat(os.path.join(path, n)).st_uid != os.getuid():
                continue
        except OSError:
            continue
        out.setdefault(m.group(1), []).append(n)
    return out


def sweep_orphans(path: str = "/dev/shm", pid_alive=None) -> int:
    """Removes what `orphan_segments` lists; returns the number of files removed.  The launcher calls it at start
    when `LLB_SWEEP_ORPHAN_SHM=1`: the check goes by process ids, so it must stay off where several containers
    with process-id namespaces of their own share one /dev/shm."""
    n = 0
    for files in orphan_segments(path, pid_alive).values():
        for f in files:
            try:
                os.unlink(os.path.join(path, f))
                n += 1
            except OSError:
                pass
    return n


def note_or_sweep_orphans(path: str = "/dev/shm") -> int:
    """At server start: sweep when asked to, else say what lies around."""
    if os.environ.get("LLB_SWEEP_ORPHAN_SHM", "").strip().lower() in ("1", "true", "on"):
        n = sweep_orphans(path)
        if n:
            log.warning("removed %d shared-memory segments of servers that no longer run", n)
        return n
    found = orphan_segments(path)
    if found:
        log.warning("%d shared-memory segments of %d servers that no longer run lie in %s "
                    "(LLB_SWEEP_ORPHAN_SHM=1, or python -m lightllm_b200.utils.shm_cleanup --sweep, removes them)",
                    sum(len(v) for v in found.values()), len(found), path)
    return 0


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser(description="segments of servers that were killed")
    ap.add_argument("--path", default="/dev/shm")
    ap.add_argument("--sweep", action="store_true", help="remove them (default: list)")
    a = ap.parse_args()
    if a.sweep:
        print(f"removed {sweep_orphans(a.path)} segments")
    else:
        for server, files in sorted(orphan_segments(a.path).items()):
            print(f"{server}: {len(files)} segments")
