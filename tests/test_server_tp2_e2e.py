"""The whole process tree with two model-rank processes on CPU / gloo (tensor parallel 2): launcher -> router ->
two ranks that agree on the router's mailbox generation with a host all-reduce before they act -> detokenizer ->
HTTP worker.  Greedy outputs over HTTP must equal the single-rank server's (tiny Llama: 2 layers, hidden 256,
4 q / 2 kv heads, SwiGLU 688, vocabulary 1024, fp32)."""
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


def _start(d, tp):
    port = _free_port()
    env = dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=ROOT)
    log = open(d / f"server_tp{tp}.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "lightllm_b200.server.api_server", "--model_dir", str(d), "--port",
                             str(port), "--data_type", "fp32", "--max_total_token_num", "4096",
                             "--running_max_req_size", "8", "--max_req_total_len", "256", "--tp", str(tp)],
                            env=env, stdout=log, stderr=subprocess.STDOUT, cwd=ROOT, start_new_session=True)
    url = f"http://127.0.0.1:{port}"
    t0 = time.time()
    while time.time() - t0 < 300:
        if proc.poll() is not None:
            break
        try:
            if requests.get(url + "/liveness", timeout=2).status_code == 200:
                return proc, url
        except Exception:
            time.sleep(1)
    proc.kill()
    pytest.fail(f"server --tp {tp} did not start:\n" + open(d / f"server_tp{tp}.log").read()[-3000:])


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
    for n, new in ((40, 12), (17, 8), (64, 16)):
        body = {"inputs": list(range(5, 5 + n)), "parameters": {"max_new_tokens": new, "ignore_eos": True,
                                                                "return_details": True}}
        r = requests.post(url + "/generate", json=body, timeout=120).json()
        assert r["count_output_tokens"] == new and r["finish_reason"] == "length"
        outs.append([t["id"] for t in r["tokens"]])
    # a streamed request and an aborted one: both ranks must drop it on the same step and stay usable
    with requests.post(url + "/generate_stream", json={"inputs": list(range(9, 60)), "parameters":
                                                        {"max_new_tokens": 200, "ignore_eos": True}},
                       stream=True, timeout=120) as r:
        got = 0
        for line in r.iter_lines():
            if line.startswith(b"data:"):
                got += 1
                if got == 3:
                    break          # client goes away
    r = requests.post(url + "/generate", json={"inputs": list(range(5, 45)), "parameters":
                                               {"max_new_tokens": 12, "ignore_eos": True, "return_details": True}},
                      timeout=120).json()
    outs.append([t["id"] for t in r["tokens"]])
    return outs


@pytest.mark.timeout(900)
def test_two_rank_server_matches_one_rank(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    # one rank: the offline engine on the same random weights
    from lightllm_b200.engine.llm import LLM

    llm = LLM(config=CFG, data_type="float32", max_total_token_num=4096, running_max_req_size=8, max_req_total_len=256,
              batch_max_tokens=256)
    one = [llm.generate([list(range(5, 5 + n))], {"max_new_tokens": new, "ignore_eos": True})[0]["token_ids"]
           for n, new in ((40, 12), (17, 8), (64, 16), (40, 12))]
    p2, u2 = _start(tmp_path, 2)
    try:
        two = _ask(u2)
        assert requests.get(u2 + "/health", timeout=30).status_code == 200
    finally:
        _stop(p2)
    assert two == one
    assert one[3] == one[0]          # the request after the aborted stream repeats the first one exactly
