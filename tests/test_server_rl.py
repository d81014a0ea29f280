"""RL control plane over real HTTP on a CPU server: pause / continue, cache flush, memory release / resume, and a
weight update from tensors that changes what the model generates."""
import base64
import io
import json
import os
import signal
import socket
import subprocess
import sys
import time

import pytest
import requests
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = {"model_type": "llama", "hidden_size": 128, "num_hidden_layers": 2, "num_attention_heads": 4,
       "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 256, "vocab_size": 512, "rms_norm_eps": 1e-6,
       "rope_theta": 10000.0, "eos_token_id": 2, "max_position_embeddings": 512, "torch_dtype": "float32"}


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    d = tmp_path_factory.mktemp("tiny_rl_model")
    (d / "config.json").write_text(json.dumps(CFG))
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=ROOT)
    log = open(d / "server.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "lightllm_b200.server.api_server", "--model_dir", str(d), "--port",
                             str(port), "--data_type", "fp32", "--max_total_token_num", "2048",
                             "--running_max_req_size", "4", "--max_req_total_len", "128", "--tp", "1", "--enable_rl"],
                            env=env, stdout=log, stderr=subprocess.STDOUT, cwd=ROOT, start_new_session=True)
    url = f"http://127.0.0.1:{port}"
    t0, up = time.time(), False
    while time.time() - t0 < 240 and proc.poll() is None:
        try:
            if requests.get(url + "/liveness", timeout=2).status_code == 200:
                up = True
                break
        except Exception:
            time.sleep(1)
    if not up:
        proc.kill()
        pytest.fail("server did not start:\n" + open(d / "server.log").read()[-3000:])
    yield url
    try:
        os.killpg(proc.pid, signal.SIGTERM)
    except ProcessLookupError:
        pass
    try:
        proc.wait(timeout=20)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)


def _gen(url, n=6):
    body = {"inputs": list(range(5, 25)), "parameters": {"max_new_tokens": n, "ignore_eos": True, "return_details": True}}
    return requests.post(url + "/generate", json=body, timeout=60)


@pytest.mark.timeout(600)
def test_pause_flush_release_and_weight_update(server):
    first = _gen(server).json()
    assert first["count_output_tokens"] == 6
    assert _gen(server).json()["tokens"][0]["prompt_cache_len"] >= 16          # the prefix cache holds the prompt
    assert requests.post(server + "/flush_cache", timeout=30).json()["success"]
    assert _gen(server).json()["tokens"][0]["prompt_cache_len"] == 0           # ... and was emptied
    assert requests.post(server + "/pause_generation", timeout=30).json()["success"]
    assert _gen(server).status_code != 200                                     # admission is closed
    assert requests.post(server + "/continue_generation", timeout=30).json()["success"]
    assert _gen(server).status_code == 200
    assert requests.post(server + "/release_memory_occupation", json={"tags": ["kv_cache"]}, timeout=60).json()["success"]
    assert requests.post(server + "/resume_memory_occupation", json={"tags": ["kv_cache"]}, timeout=60).json()["success"]
    again = _gen(server).json()
    assert again["generated_text"] == first["generated_text"]                  # same weights, same greedy text

    def pack(t):
        buf = io.BytesIO()
        torch.save(t, buf)
        return base64.b64encode(buf.getvalue()).decode()

    new_head = torch.randn(512, 128, generator=torch.Generator().manual_seed(7)) * 0.05
    r = requests.post(server + "/update_weights_from_tensor",
                      json={"named_tensors": [["lm_head.weight", pack(new_head)]], "weight_version": "v2"}, timeout=120)
    assert r.status_code == 200 and r.json()["success"], r.text
    assert requests.get(server + "/get_weight_version", timeout=10).json().get("weight_version") == "v2"
    changed = _gen(server).json()
    assert changed["count_output_tokens"] == 6 and changed["generated_text"] != first["generated_text"]
    assert requests.post(server + "/abort_request", json={"abort_all": True}, timeout=30).json()["success"]
