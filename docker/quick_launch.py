"""Builds the `docker run` command line for a serving container and runs it (or prints it with --dry_run).

    python docker/quick_launch.py --model_dir /data/Llama-3-8B --tp 1 --port 8000 -- --max_total_token_num 400000

Everything after `--` goes to `lightllm_b200.server.api_server` unchanged.  The model directory is mounted
read-only at the same path; all GPUs are visible; /dev/shm is sized with --shm_size.
Reference: tools/quick_launch_docker.py.
"""
from __future__ import annotations

import argparse
import os
import shlex
import subprocess
import sys


def build_command(a, passthrough):
    model = os.path.abspath(a.model_dir)
    cmd = ["docker", "run", "--rm", "--gpus", a.gpus, "--shm-size", a.shm_size, "--ipc", "host" if a.host_ipc else "private",
           "-p", f"{a.port}:{a.port}", "-v", f"{model}:{model}:ro"]
    if a.name:
        cmd += ["--name", a.name]
    for e in a.env or []:
        cmd += ["-e", e]
    if a.detach:
        cmd.append("-d")
    cmd += [a.image, "python", "-m", "lightllm_b200.server.api_server", "--model_dir", model, "--tp", str(a.tp),
            "--host", "0.0.0.0", "--port", str(a.port)] + list(passthrough)
    return cmd


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    extra = []
    if "--" in argv:
        i = argv.index("--")
        argv, extra = argv[:i], argv[i + 1:]
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_dir", required=True)
    ap.add_argument("--image", default="lightllm-b200")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--gpus", default="all")
    ap.add_argument("--shm_size", default="32g")
    ap.add_argument("--name", default=None)
    ap.add_argument("--env", "-e", action="append")
    ap.add_argument("--host_ipc", action="store_true")
    ap.add_argument("--detach", "-d", action="store_true")
    ap.add_argument("--dry_run", action="store_true")
    a = ap.parse_args(argv)
    cmd = build_command(a, extra)
    print(" ".join(shlex.quote(c) for c in cmd))
    if not a.dry_run:
        return subprocess.call(cmd)
    return 0


if __name__ == "__main__":
    sys.exit(main())
