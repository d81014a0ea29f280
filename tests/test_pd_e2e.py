"""Prefill / decode disaggregation end to end on CPU: a pd_master, one prefill node and one decode node (each a
complete server with its own router and model rank), KV pages over gloo.  The tokens a client gets from the
master equal those of the offline engine on the same weights."""
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
CFG = {"model_type": "llama", "hidden_size": 128, "num_hidden_layers": 2, "num_attention_heads": 4,
       "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 256, "vocab_size": 512, "rms_norm_eps": 1e-6,
       "rope_theta": 10000.0, "eos_token_id": 2, "max_position_embeddings": 512, "torch_dtype": "float32"}


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _spawn(args, log_path):
    env = dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=ROOT)
    log = open(log_path, "w")
    return subprocess.Popen([sys.executable, "-m", "lightllm_b200.server.api_server"] + args, env=env, stdout=log,
                            stderr=subprocess.STDOUT, cwd=ROOT, start_new_session=True)


def _wait_up(url, proc, log_path, seconds=240):
    t0 = time.time()
    while time.time() - t0 < seconds:
        if proc.poll() is not None:
            break
        try:
            if requests.get(url + "/liveness", timeout=2).status_code == 200:
                return
        except Exception:
            time.sleep(1)
    pytest.fail(f"{url} did not start:\n" + open(log_path).read()[-3000:])


@pytest.fixture(scope="module")
def cluster(tmp_path_factory):
    d = tmp_path_factory.mktemp("pd")
    (d / "config.json").write_text(json.dumps(CFG))
    pm, pp, pdp = _free_port(), _free_port(), _free_port()
    procs = []
    common = ["--model_dir", str(d), "--data_type", "fp32", "--max_total_token_num", "4096", "--running_max_req_size", "8",
              "--max_req_total_len", "256", "--tp", "1", "--host", "127.0.0.1"]
    try:
        master = _spawn(["--run_mode", "pd_master", "--port", str(pm), "--host", "127.0.0.1", "--model_dir", str(d),
                         "--select_p_d_node_strategy", "round_robin"], d / "master.log")
        procs.append(master)
        _wait_up(f"http://127.0.0.1:{pm}", master, d / "master.log")
        pd_flags = ["--pd_master_ip", "127.0.0.1", "--pd_master_port", str(pm), "--pd_kv_page_size", "16"]
        prefill = _spawn(common + ["--run_mode", "prefill", "--port", str(pp)] + pd_flags, d / "prefill.log")
        decode = _spawn(common + ["--run_mode", "decode", "--port", str(pdp)] + pd_flags, d / "decode.log")
        procs += [prefill, decode]
        _wait_up(f"http://127.0.0.1:{pp}", prefill, d / "prefill.log")
        _wait_up(f"http://127.0.0.1:{pdp}", decode, d / "decode.log")
        yield {"master": f"http://127.0.0.1:{pm}", "dir": d}
    finally:
        for p in procs:
            try:
                os.killpg(p.pid, signal.SIGTERM)
            except ProcessLookupError:
                pass
        for p in procs:
            try:
                p.wait(timeout=20)
            except subprocess.TimeoutExpired:
                os.killpg(p.pid, signal.SIGKILL)


@pytest.mark.timeout(900)
def test_pd_generate_matches_offline(cluster):
    from lightllm_b200.engine.llm import LLM

    url, d = cluster["master"], cluster["dir"]
    prompt = list(range(7, 60))
    t0 = time.time()
    r = None
    while time.time() - t0 < 60:   # the nodes register with the master a moment after they come up
        r = requests.post(url + "/generate", json={"inputs": prompt, "parameters": {
            "max_new_tokens": 9, "ignore_eos": True, "return_details": True}}, timeout=120)
        if r.status_code == 200:
            break
        time.sleep(2)
    logs = "\n".join(f"--- {n}\n" + open(d / n).read()[-1500:] for n in ("master.log", "prefill.log", "decode.log"))
    assert r is not None and r.status_code == 200, (r.text if r is not None else "") + logs
    out = r.json()
    assert out["count_output_tokens"] == 9 and out["finish_reason"] == "length", str(out) + logs
    got = [t["id"] for t in out["tokens"]]
    llm = LLM(config=CFG, data_type="float32", max_total_token_num=2048, running_max_req_size=4, max_req_total_len=256,
              batch_max_tokens=256)
    want = llm.generate([prompt], {"max_new_tokens": 9, "ignore_eos": True})[0]["token_ids"]
    assert got == want, logs


@pytest.mark.timeout(900)
def test_clients_that_leave_mid_stream_leak_nothing(cluster):
    """Streams through the master, some clients hang up after one, two or five tokens (before or after the KV has
    moved to the decode node); afterwards more sequential requests than either node has request slots complete."""
    import random
    import threading

    url = cluster["master"]
    for it in range(3):
        rng = random.Random(it)
        results = []

        def client():
            ids = [rng.randrange(3, 500) for _ in range(rng.randrange(20, 80))]
            leave = rng.choice([1, 2, 5, None])
            got, t0 = 0, time.time()
            try:
                with requests.post(url + "/generate_stream", json={"inputs": ids, "parameters": {
                        "max_new_tokens": 30, "ignore_eos": True}}, stream=True, timeout=120) as r:
                    assert r.status_code == 200, r.text
                    for line in r.iter_lines():
                        if line.startswith(b"data:"):
                            got += 1
                            if leave is not None and got >= leave:
                                break
                results.append((got, leave, time.time() - t0))
            except Exception as e:  # noqa: BLE001
                results.append(("error", repr(e), time.time() - t0))

        threads = [threading.Thread(target=client) for _ in range(6)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=150)
        assert len(results) == 6 and all(r[0] != "error" for r in results), results
        assert all(r[0] == (30 if r[1] is None else r[1]) for r in results), results
    for k in range(10):           # 8 request slots per node: a leaked slot would show here
        r = requests.post(url + "/generate", json={"inputs": list(range(5 + k, 40 + k)), "parameters": {
            "max_new_tokens": 4, "ignore_eos": True}}, timeout=120)
        assert r.status_code == 200 and r.json()["count_output_tokens"] == 4, r.text
