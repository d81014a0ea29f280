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


def port_is_free(host: str, port: int) -> bool:
    """Whether a listening socket can be bound to (host, port) right now."""
    s = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
    s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    try:
        s.bind((host if host not in (None, "") else "0.0.0.0", int(port)))
        return True
    except OSError:
        return False
    finally:
        s.close()


def require_free_ports(host: str, ports, what: str = "server"):
    """Stops with one clear line before any process is started (the HTTP server would only find out at the end of
    start-up).  Reference: lightllm/server/api_start.py (validate_ports)."""
    busy = [int(p) for p in ports if p is not None and not port_is_free(host, p)]
    if busy:
        raise SystemExit(f"[lightllm_b200] cannot start the {what}: port(s) {busy} on {host or '0.0.0.0'} are in use")
