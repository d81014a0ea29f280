"""Small liveness and bookkeeping helpers used by the server processes.

`Watchdog`: a daemon thread that calls `on_timeout` (default: exit the process with status 1) when `heartbeat()`
has not been called for `timeout` seconds.  `TimeChecker`: true once per `threshold` seconds.  `MovingAverage`:
running mean with a rate-limited log line.  `retry`: decorator that repeats a call that raised.

Reference: lightllm/utils/watchdog_utils.py, time_utils.py, statics_utils.py, retry_utils.py.
"""
from __future__ import annotations

import functools
import logging
import os
import threading
import time
from typing import Callable, Optional

log = logging.getLogger(__name__)


class Watchdog:
    def __init__(self, timeout: float, on_timeout: Optional[Callable[[], None]] = None, poll: float = 2.0):
        self.timeout = float(timeout)
        self.poll = float(poll)
        self.on_timeout = on_timeout or self._exit
        self._last = time.monotonic()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.fired = 0

    @staticmethod
    def _exit():
        log.error("watchdog: no heartbeat, leaving")
        os._exit(1)

    def start(self):
        self._last = time.monotonic()
        self._thread = threading.Thread(target=self._run, name="watchdog", daemon=True)
        self._thread.start()
        return self

    def _run(self):
        while not self._stop.wait(self.poll):
            if time.monotonic() - self._last > self.timeout:
                self.fired += 1
                self._last = time.monotonic()  # one call per missed period, not one per poll
                self.on_timeout()

    def heartbeat(self):
        self._last = time.monotonic()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=self.poll + 1.0)


class TimeChecker:
    """`has_exceeded()` is true at most once per `threshold` seconds (used to rate-limit periodic work)."""

    def __init__(self, threshold: float):
        self.threshold = float(threshold)
        self._t0 = time.monotonic()

    def has_exceeded(self) -> bool:
        now = time.monotonic()
        if now - self._t0 > self.threshold:
            self._t0 = now
            return True
        return False


class MovingAverage:
    def __init__(self, log_every_s: float = 30.0):
        self.total = 0.0
        self.count = 0
        self._gate = TimeChecker(log_every_s)

    def add(self, value: float):
        self.total += float(value)
        self.count += 1

    def average(self) -> float:
        return self.total / self.count if self.count else 0.0

    def print_log(self, what: str):
        if self._gate.has_exceeded():
            log.info("%s: %.4f over %d samples", what, self.average(), self.count)


def retry(max_attempts: int = 3, wait_time: float = 1.0, exceptions=(Exception,)):
    """Calls the function up to `max_attempts` times; the last failure is re-raised with the earlier one chained."""

    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*a, **kw):
            last = None
            for attempt in range(1, max_attempts + 1):
                try:
                    return fn(*a, **kw)
                except exceptions as e:  # noqa: PERF203
                    last = e
                    log.warning("%s failed (%d/%d): %s", fn.__name__, attempt, max_attempts, e)
                    if attempt < max_attempts:
                        time.sleep(wait_time)
            raise RuntimeError(f"{fn.__name__} failed {max_attempts} times") from last

        return wrapper

    return deco
