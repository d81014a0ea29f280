"""Loggers of the server processes.

`init_logger(name)` returns a logger that writes `LEVEL time [name:line] message` lines to standard output (the
launcher's children inherit it, so one stream carries the whole server) and, when `LIGHTLLM_LOG_DIR` is set, also
to `<dir>/<process title or pid>.log`.  The level comes from `LIGHTLLM_LOG_LEVEL` (alias `LLB_LOG_LEVEL`; names or
numbers, default `info`).  Reference: lightllm/utils/log_utils.py.
"""
from __future__ import annotations

import logging
import os
import sys
import threading
from typing import Dict

_FORMAT = "%(levelname)s %(asctime)s [%(name)s:%(lineno)d] %(message)s"
_DATE = "%m-%d %H:%M:%S"
_lock = threading.Lock()
_loggers: Dict[str, logging.Logger] = {}
_root_ready = False


def log_level() -> int:
    raw = os.environ.get("LLB_LOG_LEVEL", os.environ.get("LIGHTLLM_LOG_LEVEL", "info")).strip()
    if raw.isdigit():
        return int(raw)
    return getattr(logging, raw.upper(), logging.INFO) if isinstance(getattr(logging, raw.upper(), None), int) \
        else logging.INFO


def _setup_root():
    global _root_ready
    if _root_ready:
        return
    root = logging.getLogger("lightllm_b200")
    root.setLevel(log_level())
    root.propagate = False
    fmt = logging.Formatter(_FORMAT, datefmt=_DATE)
    out = logging.StreamHandler(sys.stdout)
    out.setFormatter(fmt)
    root.addHandler(out)
    log_dir = os.environ.get("LLB_LOG_DIR", os.environ.get("LIGHTLLM_LOG_DIR"))
    if log_dir:
        try:
            os.makedirs(log_dir, exist_ok=True)
            fh = logging.FileHandler(os.path.join(log_dir, f"pid{os.getpid()}.log"))
            fh.setFormatter(fmt)
            root.addHandler(fh)
        except OSError as e:
            root.warning("cannot write logs under %s: %s", log_dir, e)
    _root_ready = True


def init_logger(name: str) -> logging.Logger:
    """A child of the package logger named after the module (`lightllm_b200.` is cut off for brevity)."""
    with _lock:
        _setup_root()
        short = name[len("lightllm_b200."):] if name.startswith("lightllm_b200.") else name
        lg = _loggers.get(short)
        if lg is None:
            lg = _loggers[short] = logging.getLogger("lightllm_b200." + short)
        return lg


def reset_for_tests():
    global _root_ready
    with _lock:
        root = logging.getLogger("lightllm_b200")
        for h in list(root.handlers):
            root.removeHandler(h)
            h.close()
        _root_ready = False
        _loggers.clear()
