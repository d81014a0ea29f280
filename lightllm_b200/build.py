"""In-tree build of the native code (sm_100a CUDA kernels and the C++ runtime pieces).

    python -m lightllm_b200.build            # build what is stale
    python -m lightllm_b200.build --force    # rebuild everything

Each ``csrc/*.cu`` is compiled to an object with
``nvcc -gencode arch=compute_100a,code=sm_100a`` and linked into
``lightllm_b200/_lib/libllb_kernels.so``; each ``csrc/runtime/*.cpp`` goes into
``lightllm_b200/_lib/libllb_runtime.so`` (host-only: shared-memory atomics, slot allocator,
radix tree).  The libraries export a C ABI and are loaded with ctypes, so there is no
dependency on the PyTorch C++ ABI and a cross-compile on a machine without a GPU works.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "_lib"
OBJ = LIB / "obj"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
    "-Xptxas",
    "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(str(p.name).encode())
        h.update(Path(p).read_bytes())
    return h.hexdigest()


def _compile_cu(src: Path, headers, force: bool, debug_bounds: bool = False) -> Path:
    tag = ".dbg" if debug_bounds else ""
    flags = NVCC_FLAGS + (["-DLLB_DEBUG_BOUNDS"] if debug_bounds else [])
    obj = OBJ / (src.stem + tag + ".o")
    stamp = OBJ / (src.stem + tag + ".sha")
    dig = _digest([src, *headers]) + " ".join(flags)
    if not force and obj.exists() and stamp.exists() and stamp.read_text() == dig:
        return obj
    cmd = [_nvcc(), *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    (OBJ / (src.stem + tag + ".ptxas.log")).write_text(r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stderr[-6000:]}")
    stamp.write_text(dig)
    return obj


def build_kernels(force: bool = False, verbose: bool = True, debug_bounds: bool = False) -> Path:
    """`debug_bounds`: the variant with index checks (-DLLB_DEBUG_BOUNDS, see csrc/common.cuh), linked into
    libllb_kernels_dbg.so; it is loaded instead of the regular library when LLB_DEBUG_BOUNDS=1 at run time."""
    OBJ.mkdir(parents=True, exist_ok=True)
    srcs = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    out = LIB / ("libllb_kernels_dbg.so" if debug_bounds else "libllb_kernels.so")
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs) or 1)) as ex:
        objs = list(ex.map(lambda s: _compile_cu(s, headers, force, debug_bounds), srcs))
    link_stamp = OBJ / ("link.dbg.sha" if debug_bounds else "link.sha")
    dig = _digest(objs)
    if force or not out.exists() or not link_stamp.exists() or link_stamp.read_text() != dig:
        cmd = [_nvcc(), "-shared", "-o", str(out), *map(str, objs), "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stderr[-4000:]}")
        link_stamp.write_text(dig)
        if verbose:
            print(f"[build] linked {out} from {len(objs)} objects")
    return out


def build_runtime(force: bool = False, verbose: bool = True) -> Path:
    LIB.mkdir(parents=True, exist_ok=True)
    OBJ.mkdir(parents=True, exist_ok=True)
    srcs = sorted((CSRC / "runtime").glob("*.cpp"))
    out = LIB / "libllb_runtime.so"
    if not srcs:
        return out
    headers = sorted((CSRC / "runtime").glob("*.h"))
    stamp = OBJ / "runtime.sha"
    dig = _digest([*srcs, *headers]) + " ".join(CXX_FLAGS)
    if not force and out.exists() and stamp.exists() and stamp.read_text() == dig:
        return out
    cxx = os.environ.get("CXX", "g++")
    cmd = [cxx, *CXX_FLAGS, "-I", str(CSRC / "runtime"), *map(str, srcs), "-o", str(out), "-lrt"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed:\n{r.stderr[-6000:]}")
    stamp.write_text(dig)
    if verbose:
        print(f"[build] built {out}")
    return out


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel as printed by ``-Xptxas -v``."""
    parts = []
    for log in sorted(OBJ.glob("*.ptxas.log")):
        parts.append(f"== {log.stem}\n{log.read_text()}")
    return "\n".join(parts)


def build_all(force: bool = False, verbose: bool = True):
    out = build_kernels(force, verbose), build_runtime(force, verbose)
    if os.environ.get("LLB_DEBUG_BOUNDS", "0") == "1":
        build_kernels(force, verbose, debug_bounds=True)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--report", action="store_true", help="print the ptxas resource report")
    a = ap.parse_args()
    build_all(a.force)
    if a.report:
        sys.stdout.write(ptxas_report())
