"""Two-node tensor parallelism on one host (CPU / gloo): two launchers (`--nnodes 2`, one model rank each) whose
routers agree on every message to their ranks (`router/multinode_sync.py`) while node 0's HTTP server relays the
requests to node 1 (`httpserver/multinode_relay.py`).  Outputs equal a single-node server's; a client that goes away
in mid-stream (known to node 0 only) is dropped on both nodes and the pair stays in lock-step afterwards.
Reference: lightllm/server/router/multinode_tp_helper.py, test/start_scripts/multi_node_tp_node0.sh / node1.sh."""
import json
import os
import signal
import socket
import subprocess
import sys
import time

import pytest
import requests

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = {"model_type": "llama", "hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 4,
       "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 688, "vocab_size": 1024, "rms_norm_eps": 1e-6,
       "rope_theta": 10000.0, "eos_token_id": 2, "max_position_embeddings": 512, "torch_dtype": "float32"}


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _launch(d, tag, port, extra):
    env = dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=ROOT)
    log = open(d / f"{tag}.log", "w")
    return subprocess.Popen([sys.executable, "-m", "lightllm_b200.server.api_server", "--model_dir", str(d), "--port",
                             str(port), "--data_type", "fp32", "--max_total_token_num", "4096",
                             "--running_max_req_size", "8", "--max_req_total_len", "256"] + extra,
                            env=env, stdout=log, stderr=subprocess.STDOUT, cwd=ROOT, start_new_session=True)


def _wait(url, procs, d, timeout_s=300):
    t0 = time.time()
    while time.time() - t0 < timeout_s:
        if any(p.poll() is not None for p in procs):
            break
        try:
            if requests.get(url + "/liveness", timeout=2).status_code == 200:
                return
        except Exception:
            time.sleep(1)
    for p in procs:
        _stop(p)
    logs = "\n".join(f"== {f.name}\n" + f.read_text()[-1500:] for f in sorted(d.glob("*.log")))
    pytest.fail("servers did not start:\n" + logs)


def _stop(proc):
    try:
        os.killpg(proc.pid, signal.SIGTERM)
    except ProcessLookupError:
        return
    try:
        proc.wait(timeout=20)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)


def _ask(url):
    outs = []
    for n, new in ((40, 10), (17, 6), (64, 12)):
        body = {"inputs": list(range(5, 5 + n)), "parameters": {"max_new_tokens": new, "ignore_eos": True,
                                                                "return_details": True}}
        r = requests.post(url + "/generate", json=body, timeout=120).json()
        assert r["count_output_tokens"] == new
        outs.append([t["id"] for t in r["tokens"]])
    return outs


@pytest.mark.timeout(900)
def test_two_nodes_on_one_host(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    # what a single rank produces for the same requests (the offline engine on the same random weights)
    from lightllm_b200.engine.llm import LLM

    llm = LLM(config=CFG, data_type="float32", max_total_token_num=4096, running_max_req_size=8, max_req_total_len=256,
              batch_max_tokens=256)
    want = [llm.generate([list(range(5, 5 + n))], {"max_new_tokens": new, "ignore_eos": True})[0]["token_ids"]
            for n, new in ((40, 10), (17, 6), (64, 12))]
    http0, http1, nccl, relay, gloo = (_free_port() for _ in range(5))
    common = ["--tp", "2", "--nnodes", "2", "--nccl_host", "127.0.0.1", "--nccl_port", str(nccl),
              "--multinode_httpmanager_port", str(relay), "--multinode_router_gloo_port", str(gloo)]
    nodes = [_launch(tmp_path, "node0", http0, common + ["--node_rank", "0"]),
             _launch(tmp_path, "node1", http1, common + ["--node_rank", "1"])]
    url = f"http://127.0.0.1:{http0}"
    try:
        _wait(url, nodes, tmp_path)
        got = _ask(url)
        assert got == want                                # fp32: tensor parallel over two nodes = one rank
        # a client that leaves in mid-stream: only node 0 sees it, both nodes must drop the request
        with requests.post(url + "/generate_stream", json={"inputs": list(range(9, 60)), "parameters":
                                                           {"max_new_tokens": 200, "ignore_eos": True}},
                           stream=True, timeout=120) as r:
            seen = 0
            for line in r.iter_lines():
                if line.startswith(b"data:"):
                    seen += 1
                    if seen == 3:
                        break
        time.sleep(2)
        assert _ask(url) == want                          # still in lock-step (prefix-cache hits on both nodes)
        # more requests than request slots (8): finished requests are recycled on BOTH nodes (every node's first
        # rank publishes tokens and finish states into its own node's request objects)
        for i in range(12):
            r = requests.post(url + "/generate", json={"inputs": list(range(5 + i, 30 + i)), "parameters":
                                                       {"max_new_tokens": 3, "ignore_eos": True}}, timeout=60)
            assert r.status_code == 200 and r.json()["count_output_tokens"] == 3, (i, r.text[:200])
        assert all(p.poll() is None for p in nodes)
    finally:
        for p in nodes:
            _stop(p)


@pytest.mark.timeout(900)
def test_losing_a_node_takes_the_other_one_down(tmp_path):
    """One tensor-parallel group over two nodes cannot go on without one of them: when node 1 is killed, node 0's
    ranks fail in their next collective, its launcher ends the whole server (a supervisor restarts both) and the
    open streams end instead of hanging."""
    import threading

    (tmp_path / "config.json").write_text(json.dumps(CFG))
    http0, http1, nccl, relay, gloo = (_free_port() for _ in range(5))
    common = ["--tp", "2", "--nnodes", "2", "--nccl_host", "127.0.0.1", "--nccl_port", str(nccl),
              "--multinode_httpmanager_port", str(relay), "--multinode_router_gloo_port", str(gloo)]
    nodes = [_launch(tmp_path, "node0", http0, common + ["--node_rank", "0"]),
             _launch(tmp_path, "node1", http1, common + ["--node_rank", "1"])]
    url = f"http://127.0.0.1:{http0}"
    try:
        _wait(url, nodes, tmp_path)
        ended, streaming = [], threading.Event()

        def client():
            got = 0
            try:
                with requests.post(url + "/generate_stream", json={"inputs": list(range(5, 60)), "parameters": {
                        "max_new_tokens": 240, "ignore_eos": True}}, stream=True, timeout=300) as r:
                    for line in r.iter_lines():
                        if line.startswith(b"data:"):
                            got += 1
                            if got == 3:
                                streaming.set()
                ended.append(("closed", got))
            except Exception as e:  # noqa: BLE001
                ended.append((type(e).__name__, got))

        t = threading.Thread(target=client)
        t.start()
        assert streaming.wait(120)
        os.killpg(nodes[1].pid, signal.SIGKILL)
        t0 = time.time()
        while time.time() - t0 < 180 and nodes[0].poll() is None:
            time.sleep(1)
        assert nodes[0].poll() is not None, "node 0 kept running without its peer"
        t.join(timeout=60)
        assert ended and ended[0][1] < 240, ended
        assert "shutting everything down" in (tmp_path / "node0.log").read_text()
    finally:
        for p in nodes:
            _stop(p)
