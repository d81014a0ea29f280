"""`--enable_prompt_logprobs`: `/generate` with `prompt_logprobs` = 0 returns every prompt token's logprob and rank,
with k > 0 also the k most likely tokens per position (whole server on CPU).
Reference: lightllm/server/core/objs/token_metadata.py:100-157, lightllm/server/api_lightllm.py:70-112."""
import json
import math
import os
import signal
import socket
import subprocess
import sys
import time

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


@pytest.mark.timeout(600)
def test_prompt_logprobs_over_http(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    port = _free_port()
    env = dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=ROOT)
    log = open(tmp_path / "server.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "lightllm_b200.server.api_server", "--model_dir", str(tmp_path),
                             "--port", str(port), "--data_type", "fp32", "--max_total_token_num", "2048",
                             "--running_max_req_size", "4", "--max_req_total_len", "128", "--tp", "1",
                             "--enable_prompt_logprobs"],
                            env=env, stdout=log, stderr=subprocess.STDOUT, cwd=ROOT, start_new_session=True)
    url = f"http://127.0.0.1:{port}"
    try:
        t0, up = time.time(), False
        while time.time() - t0 < 240 and proc.poll() is None:
            try:
                if requests.get(url + "/liveness", timeout=2).status_code == 200:
                    up = True
                    break
            except Exception:
                time.sleep(1)
        assert up, open(tmp_path / "server.log").read()[-3000:]
        ids = list(range(7, 37))
        body = {"inputs": ids, "parameters": {"max_new_tokens": 3, "ignore_eos": True, "prompt_logprobs": 0}}
        r0 = requests.post(url + "/generate", json=body, timeout=120).json()
        assert r0["prompt_token_ids"] == ids and len(r0["prompt_logprobs"]) == 30 and r0["prompt_logprobs"][0] is None
        own = []
        for pos in range(1, 30):
            entry = r0["prompt_logprobs"][pos]
            assert list(entry) == [str(ids[pos])]
            e = entry[str(ids[pos])]
            assert e["logprob"] < 0 and 1 <= e["rank"] <= 512
            own.append((e["logprob"], e["rank"]))
        body["parameters"]["prompt_logprobs"] = 3
        r3 = requests.post(url + "/generate", json=body, timeout=120).json()        # no prefix-cache shortcut
        for pos in range(1, 30):
            entry = r3["prompt_logprobs"][pos]
            e = entry[str(ids[pos])]
            assert abs(e["logprob"] - own[pos - 1][0]) < 1e-4 and e["rank"] == own[pos - 1][1]
            top = sorted((v for v in entry.values() if v["rank"] <= 3), key=lambda v: v["rank"])
            assert [v["rank"] for v in top][:3] == [1, 2, 3] and len(entry) in (3, 4)
            assert top[0]["logprob"] >= top[1]["logprob"] >= top[2]["logprob"] >= e["logprob"] - 1e-6 or e["rank"] <= 3
            assert math.exp(top[0]["logprob"]) <= 1.0
        plain = requests.post(url + "/generate", json={"inputs": ids, "parameters": {"max_new_tokens": 3}},
                              timeout=120).json()
        assert "prompt_logprobs" not in plain
    finally:
        try:
            os.killpg(proc.pid, signal.SIGTERM)
        except ProcessLookupError:
            pass
        try:
            proc.wait(timeout=20)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)
