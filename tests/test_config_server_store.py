"""`--use_config_server_to_init_nccl`: the rendezvous store of a model world lives in the config server; every rank
(rank 0 included) joins it as a client.  Two gloo ranks on one host.
Reference: lightllm/utils/dist_utils.py:293-318, lightllm/server/config_server/api_http.py:163-215."""
import os
import signal
import socket
import subprocess
import sys
import time

import pytest
import requests
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, http_port, store_port, out_dir):
    import torch.distributed as dist

    from lightllm_b200.parallel import dist as pdist

    if rank == 1:
        time.sleep(1.0)        # rank 0 asks first; an early rank just polls
    ps = pdist.init_distributed(2, rank, host="127.0.0.1", port=store_port, backend="gloo", device=torch.device("cpu"),
                                config_server=("127.0.0.1", http_port))
    t = torch.tensor([rank + 1.0])
    dist.all_reduce(t)
    open(os.path.join(out_dir, f"r{rank}"), "w").write(f"{float(t)} {os.environ.get('TORCHELASTIC_USE_AGENT_STORE')} "
                                                       f"{ps.world_size}")
    pdist.destroy()


@pytest.mark.timeout(300)
def test_ranks_rendezvous_through_the_config_server(tmp_path):
    http_port, store_port = _free_port(), _free_port()
    env = dict(os.environ, PYTHONPATH=ROOT)
    log = open(tmp_path / "cfg.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "lightllm_b200.server.api_server", "--run_mode", "config_server",
                             "--config_server_host", "127.0.0.1", "--config_server_port", str(http_port)],
                            env=env, stdout=log, stderr=subprocess.STDOUT, cwd=ROOT, start_new_session=True)
    try:
        t0, up = time.time(), False
        while time.time() - t0 < 120 and proc.poll() is None:
            try:
                if requests.get(f"http://127.0.0.1:{http_port}/liveness", timeout=2).status_code == 200:
                    up = True
                    break
            except Exception:
                time.sleep(0.5)
        assert up, open(tmp_path / "cfg.log").read()[-2000:]
        mp.spawn(_rank, args=(http_port, store_port, str(tmp_path)), nprocs=2, join=True)
        for r in range(2):
            assert open(tmp_path / f"r{r}").read() == "3.0 True 2"
    finally:
        try:
            os.killpg(proc.pid, signal.SIGTERM)
        except ProcessLookupError:
            pass
        try:
            proc.wait(timeout=20)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)
