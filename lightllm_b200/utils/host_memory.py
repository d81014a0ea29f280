"""Host memory for the CPU tier of the KV cache: huge pages, NUMA placement, parallel pre-faulting and CUDA
registration.

`HostBuffer.create(nbytes, ...)` maps anonymous memory, optionally

* on explicit huge pages (`MAP_HUGETLB`; when the kernel has none reserved it falls back to regular pages with a
  transparent-huge-page hint), which shortens both the first touch and the registration of a cache of tens of GB,
* with a NUMA policy set before the first touch: `"interleave"` spreads the pages over all nodes with memory,
  `"local"` prefers the node the GPU hangs on (from the GPU's PCI entry in sysfs),
* touched by several threads, so that the pages exist before the registration walks them,
* registered with CUDA in 128 MB pieces (`cudaHostRegister`), after which copies to and from it run as pinned
  transfers.

Every step that the machine refuses (no huge pages, no permission for `mbind`, no CUDA) is recorded in
`HostBuffer.notes` and skipped; the buffer is usable either way.

Switches: `LLB_HUGE_PAGE_ENABLE=1` (alias `LIGHTLLM_HUGE_PAGE_ENABLE`) and `LLB_ENABLE_NUMA_INTERLEAVE=1` (alias
`LIGHTLLM_ENABLE_NUMA_INTERLEAVE`), `LLB_CPU_CACHE_NUMA=local|interleave`.

Reference: lightllm/utils/kv_cache_utils.py:174-345 (create_shm_kv_cache_ptr, register_shm_ptr_to_pin,
interleave_pages_across_numa_nodes), lightllm/utils/envs_utils.py:226-240.
"""
from __future__ import annotations

import ctypes
import mmap
import os
import platform
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

import numpy as np
import torch

MAP_HUGETLB = 0x40000
MADV_HUGEPAGE = 14
MPOL_PREFERRED, MPOL_INTERLEAVE = 1, 3
_SYS_MBIND = {"x86_64": 237, "aarch64": 235}
REGISTER_CHUNK = 128 << 20


def _env_on(*names: str) -> bool:
    return any(os.environ.get(n, "").strip().lower() in ("1", "true", "on", "yes") for n in names)


def huge_pages_wanted() -> bool:
    return _env_on("LLB_HUGE_PAGE_ENABLE", "LIGHTLLM_HUGE_PAGE_ENABLE")


def numa_policy_wanted() -> Optional[str]:
    p = os.environ.get("LLB_CPU_CACHE_NUMA", "").strip().lower()
    if p in ("local", "interleave"):
        return p
    return "interleave" if _env_on("LLB_ENABLE_NUMA_INTERLEAVE", "LIGHTLLM_ENABLE_NUMA_INTERLEAVE") else None


def default_huge_page_size(meminfo: str = "/proc/meminfo") -> int:
    try:
        with open(meminfo) as f:
            for line in f:
                if line.startswith("Hugepagesize:"):
                    return int(line.split()[1]) * 1024
    except (OSError, ValueError, IndexError):
        pass
    return 2 << 20


def parse_node_list(text: str) -> List[int]:
    """`0-1,4` -> [0, 1, 4] (the format of /sys/devices/system/node/has_memory)."""
    nodes: List[int] = []
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-", 1)
            nodes.extend(range(int(a), int(b) + 1))
        else:
            nodes.append(int(part))
    return nodes


def nodes_with_memory(sys_root: str = "/sys/devices/system/node") -> List[int]:
    for name in ("has_memory", "online"):
        try:
            with open(os.path.join(sys_root, name)) as f:
                nodes = parse_node_list(f.read())
            if nodes:
                return nodes
        except (OSError, ValueError):
            continue
    return []


def gpu_pci_address(device_index: int) -> Optional[str]:
    try:
        p = torch.cuda.get_device_properties(device_index)
        return f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
    except Exception:
        return None


def numa_node_of_gpu(device_index: int, sys_root: str = "/sys/bus/pci/devices") -> Optional[int]:
    """NUMA node of the GPU's PCI function, None when unknown (no CUDA, no sysfs entry, or the kernel says -1)."""
    addr = gpu_pci_address(device_index)
    return numa_node_of_pci(addr, sys_root) if addr else None


def numa_node_of_pci(bus_id: str, sys_root: str = "/sys/bus/pci/devices") -> Optional[int]:
    bus_id = bus_id.lower()
    if len(bus_id.split(":")[0]) == 8:      # NVML prints an 8-digit domain, sysfs a 4-digit one
        bus_id = bus_id[4:]
    try:
        with open(os.path.join(sys_root, bus_id, "numa_node")) as f:
            n = int(f.read().strip())
        return n if n >= 0 else None
    except (OSError, ValueError):
        return None


def _mbind(addr: int, nbytes: int, mode: int, nodes: List[int], libc=None) -> int:
    """0 on success, else errno."""
    nr = _SYS_MBIND.get(platform.machine())
    if nr is None or not nodes:
        return 38   # ENOSYS
    libc = libc or ctypes.CDLL(None, use_errno=True)
    maxnode = max(nodes) + 2
    words = (maxnode + 63) // 64
    mask = (ctypes.c_ulong * words)()
    for n in nodes:
        mask[n // 64] |= 1 << (n % 64)
    libc.syscall.restype = ctypes.c_long
    r = libc.syscall(ctypes.c_long(nr), ctypes.c_void_p(addr), ctypes.c_ulong(nbytes), ctypes.c_int(mode), mask,
                     ctypes.c_ulong(maxnode), ctypes.c_uint(0))
    return 0 if r == 0 else (ctypes.get_errno() or 1)


class HostBuffer:
    """An anonymous mapping and what was done to it.  `tensor(dtype, shape)` views it."""

    def __init__(self, mm: mmap.mmap, nbytes: int, mapped: int):
        self.mm, self.nbytes, self.mapped = mm, nbytes, mapped
        self.addr = ctypes.addressof(ctypes.c_char.from_buffer(mm))
        self.huge_pages = False
        self.numa: Optional[str] = None
        self.registered = False
        self.notes: List[str] = []

    @classmethod
    def create(cls, nbytes: int, huge_pages: bool = False, numa: Optional[str] = None, device_index: Optional[int] = None,
               register: bool = False, prefault_threads: int = 8) -> "HostBuffer":
        nbytes = int(nbytes)
        page = mmap.PAGESIZE
        buf = None
        if huge_pages:
            hp = default_huge_page_size()
            size = (nbytes + hp - 1) // hp * hp
            try:
                mm = mmap.mmap(-1, size, flags=mmap.MAP_PRIVATE | mmap.MAP_ANONYMOUS | MAP_HUGETLB)
                buf = cls(mm, nbytes, size)
                buf.huge_pages, page = True, hp
            except (OSError, ValueError) as e:
                note = (f"no explicit huge pages ({type(e).__name__}: {e}); reserve {size // hp} pages of "
                        f"{hp >> 20} MB (vm.nr_hugepages) to use them")
        if buf is None:
            size = (nbytes + page - 1) // page * page
            buf = cls(mmap.mmap(-1, size, flags=mmap.MAP_PRIVATE | mmap.MAP_ANONYMOUS), nbytes, size)
            if huge_pages:
                buf.notes.append(note)
                try:
                    buf.mm.madvise(MADV_HUGEPAGE)
                    buf.notes.append("transparent huge pages requested instead")
                except (OSError, ValueError, AttributeError):
                    pass
        if numa:
            buf._place(numa, device_index)
        buf._prefault(page, prefault_threads)
        if register:
            buf._register(device_index)
        return buf

    def _place(self, policy: str, device_index: Optional[int]):
        if policy == "interleave":
            nodes, mode = nodes_with_memory(), MPOL_INTERLEAVE
            if len(nodes) < 2:
                self.notes.append("one memory node: nothing to interleave")
                return
        else:
            node = numa_node_of_gpu(device_index) if device_index is not None else None
            if node is None:
                self.notes.append("the GPU's memory node is unknown: default placement")
                return
            nodes, mode = [node], MPOL_PREFERRED
        err = _mbind(self.addr, self.mapped, mode, nodes)
        if err:
            self.notes.append(f"mbind refused (errno {err}): default placement")
        else:
            self.numa = f"{policy}:{','.join(map(str, nodes))}"

    def _prefault(self, page: int, threads: int):
        arr = np.frombuffer(self.mm, dtype=np.uint8)
        n = max(1, int(threads))
        chunk = ((self.mapped + n - 1) // n + page - 1) // page * page

        def touch(i):
            lo, hi = i * chunk, min(self.mapped, (i + 1) * chunk)
            if lo < hi:
                arr[lo:hi:page] = 0

        with ThreadPoolExecutor(max_workers=n) as ex:
            list(ex.map(touch, range(n)))
        del arr

    def _register(self, device_index: Optional[int]):
        if not torch.cuda.is_available():
            self.notes.append("no CUDA device: not registered")
            return
        if device_index is not None:
            torch.cuda.set_device(device_index)
        rt = torch.cuda.cudart()
        done = 0
        while done < self.mapped:
            n = min(REGISTER_CHUNK, self.mapped - done)
            r = rt.cudaHostRegister(self.addr + done, n, 0)
            if int(r) != 0:
                for off in range(0, done, REGISTER_CHUNK):   # all or nothing
                    rt.cudaHostUnregister(self.addr + off)
                self.notes.append(f"cudaHostRegister failed ({r}) at byte {done}: copies run unpinned")
                return
            done += n
        self.registered = True

    def tensor(self, dtype: torch.dtype, shape) -> torch.Tensor:
        numel = int(np.prod(shape))
        esz = torch.empty((), dtype=dtype).element_size()
        assert numel * esz <= self.nbytes, "the view is larger than the buffer"
        return torch.frombuffer(self.mm, dtype=dtype, count=numel).view(*shape)

    def close(self):
        if self.registered:
            rt = torch.cuda.cudart()
            for off in range(0, self.mapped, REGISTER_CHUNK):
                rt.cudaHostUnregister(self.addr + off)
            self.registered = False
