"""ctypes loader for the in-tree native libraries.

``kernels()`` returns ``libllb_kernels.so`` (sm_100a CUDA kernels), ``runtime()`` returns
``libllb_runtime.so`` (host C++: shm atomics, slot allocator, radix tree).  A missing
library is an error on a machine with a GPU: the CUDA path never falls back silently.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIB_DIR = Path(__file__).resolve().parent.parent / "_lib"
_kernels = None
_runtime = None


class NativeError(RuntimeError):
    pass


_ERR_NAMES = {-1: "bad argument", -2: "unsupported shape/dtype", -3: "size beyond the stated maximum", -4: "driver entry point unavailable"}


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc < 0:
        raise NativeError(f"{what}: {_ERR_NAMES.get(rc, rc)}")
    raise NativeError(f"{what}: CUDA error {rc}")


def _load(name: str):
    path = _LIB_DIR / name
    if not path.exists():
        if os.environ.get("LLB_AUTOBUILD", "1") == "1":
            from .. import build as _b

            if name == "libllb_kernels.so":
                _b.build_kernels(verbose=False)
            else:
                _b.build_runtime(verbose=False)
    if not path.exists():
        raise NativeError(f"{path} is missing: run `python -m lightllm_b200.build`")
    return ctypes.CDLL(str(path))


def debug_bounds_enabled() -> bool:
    return os.environ.get("LLB_DEBUG_BOUNDS", "0") == "1"


def kernels():
    global _kernels
    if _kernels is None:
        if debug_bounds_enabled():   # the build with index checks (csrc/common.cuh)
            if not (_LIB_DIR / "libllb_kernels_dbg.so").exists():
                from .. import build as _b

                _b.build_kernels(verbose=False, debug_bounds=True)
            _kernels = _load("libllb_kernels_dbg.so")
        else:
            _kernels = _load("libllb_kernels.so")
    return _kernels


_DEBUG_UNITS = ("ops_basic", "attention", "attention_tc", "mla", "moe")


def set_debug_bounds(pool_slots: int = 0, req_rows: int = 0, r2t_cols: int = 0, num_experts: int = 0, status=None):
    """Declares the table sizes the checked build compares indices with (0 = unchecked) and the int32 device word
    that receives the code of the first violation.  A no-op in the regular build."""
    if not debug_bounds_enabled():
        return False
    lib = kernels()
    for unit in _DEBUG_UNITS:
        fn = getattr(lib, f"llb_debug_set_bounds_{unit}")
        check(fn(ctypes.c_int(pool_slots), ctypes.c_int(req_rows), ctypes.c_int(r2t_cols), ctypes.c_int(num_experts),
                 ptr(status)), f"debug_set_bounds_{unit}")
    return True


def runtime():
    global _runtime
    if _runtime is None:
        _runtime = _load("libllb_runtime.so")
    return _runtime


def have_kernels() -> bool:
    return (_LIB_DIR / "libllb_kernels.so").exists()


# ---- argument helpers ----
c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_int64 = ctypes.c_int64
c_float = ctypes.c_float


def ptr(t):
    """Device (or pinned host) pointer of a tensor, or NULL for None."""
    if t is None:
        return c_void_p(0)
    return c_void_p(t.data_ptr())


def stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def i64(v):
    return c_int64(int(v))


def f32(v):
    return c_float(float(v))
