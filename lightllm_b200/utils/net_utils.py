"""Port helpers (reference: lightllm/utils/net_utils.py)."""
from __future__ import annotations

import socket
from typing import List


def alloc_can_use_network_port(num: int = 3, used_ports: List[int] = None, start: int = 10000) -> List[int]:
    used = set(used_ports or [])
    out = []
    port = start
    while len(out) < num and port < 65535:
        if port not in used:
            with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
                try:
                    s.bind(("", port))
                    out.append(port)
                except OSError:
                    pass
        port += 1
    if len(out) < num:
        raise RuntimeError("not enough free ports")
    return out


def alloc_consecutive_ports(num: int, start: int = 30000, used_ports: List[int] = None) -> int:
    """First port of a run of `num` free consecutive ports (one per tensor-parallel rank)."""
    used = set(used_ports or [])
    base = start
    while base + num < 65535:
        ok = True
        for p in range(base, base + num):
            if p in used:
                ok = False
            else:
                with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
                    try:
                        s.bind(("", p))
                    except OSError:
                        ok = False
            if not ok:
                base = p + 1
                break
        if ok:
            return base
    raise RuntimeError("no run of free consecutive ports")


def get_hostname_ip() -> str:
    try:
        return socket.gethostbyname(socket.gethostname())
    except Exception:
        return "127.0.0.1"
