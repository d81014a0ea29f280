"""Host-side failure handling of the process tree (CPU server): when a model-rank process or the detokenizer dies,
the launcher tears the whole tree down (no half-alive server); a stopped (SIGSTOP) rank makes `/health` fail once
the health window has passed while requests are in flight; `DEBUG_HEALTHCHECK_RETURN_FAIL` forces a failure.
Reference behaviour: lightllm/utils/start_utils.py:113-160, lightllm/utils/process_check.py:29-46,
lightllm/utils/health_check.py:14-44."""
import json
import os
import signal
import socket
import subprocess
import sys
import threading
import time

import psutil
import pytest
import requests

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = {"model_type": "llama", "hidden_size": 128, "num_hidden_layers": 2, "num_attention_heads": 4,
       "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 256, "vocab_size": 512, "rms_norm_eps": 1e-6,
       "rope_theta": 10000.0, "eos_token_id": 2, "max_position_embeddings": 512, "torch_dtype": "float32"}


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _start(d, extra_env=None):
    (d / "config.json").write_text(json.dumps(CFG))
    port = _free_port()
    env = dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=ROOT, **(extra_env or {}))
    log = open(d / "server.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "lightllm_b200.server.api_server", "--model_dir", str(d), "--port",
                             str(port), "--data_type", "fp32", "--max_total_token_num", "2048",
                             "--running_max_req_size", "4", "--max_req_total_len", "256", "--tp", "1"],
                            env=env, stdout=log, stderr=subprocess.STDOUT, cwd=ROOT, start_new_session=True)
    url = f"http://127.0.0.1:{port}"
    t0 = time.time()
    while time.time() - t0 < 240 and proc.poll() is None:
        try:
            if requests.get(url + "/liveness", timeout=2).status_code == 200:
                return proc, url
        except Exception:
            time.sleep(1)
    proc.kill()
    pytest.fail("server did not start:\n" + open(d / "server.log").read()[-3000:])


def _children(proc, needle):
    out = []
    for c in psutil.Process(proc.pid).children(recursive=True):
        try:
            title = " ".join(c.cmdline()) + " " + c.name()
        except psutil.Error:
            continue
        if needle in title:
            out.append(c)
    return out


def _kill_tree(proc):
    try:
        os.killpg(proc.pid, signal.SIGKILL)
    except ProcessLookupError:
        pass


def _tree_gone(proc, timeout_s=60):
    t0 = time.time()
    while time.time() - t0 < timeout_s:
        if proc.poll() is not None:
            try:
                left = [p for p in psutil.process_iter(["pid"]) if os.getpgid(p.pid) == proc.pid]
            except (ProcessLookupError, psutil.Error):
                left = []
            if not left:
                return True
        time.sleep(0.5)
    return False


@pytest.mark.timeout(600)
@pytest.mark.parametrize("victim", ["model_infer", "detokenization"])
def test_losing_a_process_takes_the_whole_tree_down(tmp_path, victim):
    proc, url = _start(tmp_path)
    try:
        assert requests.post(url + "/generate", json={"inputs": [5, 6, 7], "parameters": {"max_new_tokens": 2}},
                             timeout=60).status_code == 200
        targets = _children(proc, victim)
        assert targets, [" ".join(c.cmdline()) for c in psutil.Process(proc.pid).children(recursive=True)]
        targets[0].kill()                                 # the exact pid of one child of this test's own server
        assert _tree_gone(proc), "the launcher kept running after one of its processes died"
        with pytest.raises(requests.exceptions.RequestException):
            requests.get(url + "/liveness", timeout=3)
    finally:
        _kill_tree(proc)


@pytest.mark.timeout(600)
def test_health_reports_a_stalled_rank_and_the_debug_switch(tmp_path):
    proc, url = _start(tmp_path, {"HEALTH_TIMEOUT": "3"})
    stopped = None
    try:
        assert requests.get(url + "/health", timeout=30).status_code == 200
        rank = _children(proc, "model_infer")[0]
        rank.suspend()                                    # SIGSTOP: the rank is alive but makes no progress
        stopped = rank
        done = []
        t = threading.Thread(target=lambda: done.append(
            requests.post(url + "/generate", json={"inputs": [5, 6, 7, 8], "parameters": {"max_new_tokens": 4}},
                          timeout=120).status_code), daemon=True)
        t.start()
        time.sleep(6)                                     # longer than the health window, a request in flight
        assert requests.get(url + "/health", timeout=30).status_code == 503
        rank.resume()
        stopped = None
        t.join(timeout=120)
        assert done == [200]
        assert requests.get(url + "/health", timeout=60).status_code == 200
    finally:
        if stopped is not None:
            try:
                stopped.resume()
            except psutil.Error:
                pass
        _kill_tree(proc)


def test_debug_switch_forces_an_unhealthy_answer(monkeypatch):
    """`DEBUG_HEALTHCHECK_RETURN_FAIL=true`: the health probe fails without touching the server (the reference's
    only built-in fault-injection hook)."""
    import asyncio
    import inspect

    from lightllm_b200.utils import health_check as hc

    monkeypatch.setenv("DEBUG_HEALTHCHECK_RETURN_FAIL", "true")
    fn = hc.health_check
    params = inspect.signature(fn).parameters
    res = fn(*([None] * len(params)))
    if inspect.isawaitable(res):
        res = asyncio.run(res)
    assert res is False


@pytest.mark.timeout(600)
def test_a_failed_start_leaves_no_processes_behind(tmp_path):
    """A model that cannot be built (unknown architecture): the launcher reports it, ends with a non-zero code and
    takes the processes that had already started with it (they used to keep it from exiting)."""
    import psutil

    (tmp_path / "config.json").write_text(json.dumps({"model_type": "no_such_architecture", "hidden_size": 64}))
    env = dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=ROOT)
    proc = subprocess.Popen([sys.executable, "-m", "lightllm_b200.server.api_server", "--model_dir", str(tmp_path), "--port",
                             str(_free_port()), "--data_type", "fp32"], env=env, stdout=subprocess.PIPE,
                            stderr=subprocess.STDOUT, text=True, cwd=ROOT, start_new_session=True)
    try:
        out, _ = proc.communicate(timeout=300)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)
        pytest.fail("the launcher did not exit after a failed start")
    assert proc.returncode not in (0, None) and "unsupported model_type 'no_such_architecture'" in out
    time.sleep(1)
    left = [p for p in psutil.process_iter(["cmdline", "name"]) if str(tmp_path) in " ".join(p.info["cmdline"] or [])]
    assert not left, left
    # a directory without a model: one line, at once
    r = subprocess.run([sys.executable, "-m", "lightllm_b200.server.api_server", "--model_dir", str(tmp_path / "nothing"),
                        "--port", str(_free_port())], env=env, capture_output=True, text=True, timeout=120, cwd=ROOT)
    assert r.returncode != 0 and "no config.json there" in (r.stdout + r.stderr)
