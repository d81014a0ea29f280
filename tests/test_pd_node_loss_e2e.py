"""A decode node dies while it streams (its whole process group is killed from the host): the clients' streams end
with an error at once, the master refuses requests while no decode node is registered, and serves again as soon as a
new one has registered; the prefill node and the master live through it."""
import json
import os
import signal
import subprocess
import threading
import time

import pytest
import requests

from test_pd_e2e import CFG, _free_port, _spawn, _wait_up


@pytest.mark.timeout(1200)
def test_decode_node_lost_and_replaced(tmp_path):
    d = tmp_path
    (d / "config.json").write_text(json.dumps(CFG))
    pm, pp, pd1, pd2 = _free_port(), _free_port(), _free_port(), _free_port()
    common = ["--model_dir", str(d), "--data_type", "fp32", "--max_total_token_num", "4096", "--running_max_req_size", "8",
              "--max_req_total_len", "512", "--tp", "1", "--host", "127.0.0.1"]
    procs = []
    try:
        master = _spawn(["--run_mode", "pd_master", "--port", str(pm), "--host", "127.0.0.1", "--model_dir", str(d),
                         "--select_p_d_node_strategy", "round_robin"], d / "master.log")
        procs.append(master)
        _wait_up(f"http://127.0.0.1:{pm}", master, d / "master.log")
        flags = ["--pd_master_ip", "127.0.0.1", "--pd_master_port", str(pm), "--pd_kv_page_size", "16"]
        prefill = _spawn(common + ["--run_mode", "prefill", "--port", str(pp)] + flags, d / "prefill.log")
        decode = _spawn(common + ["--run_mode", "decode", "--port", str(pd1)] + flags, d / "decode.log")
        procs += [prefill, decode]
        _wait_up(f"http://127.0.0.1:{pp}", prefill, d / "prefill.log")
        _wait_up(f"http://127.0.0.1:{pd1}", decode, d / "decode.log")
        url = f"http://127.0.0.1:{pm}"
        t0 = time.time()
        while time.time() - t0 < 60:       # registration follows a moment after start-up
            if requests.post(url + "/generate", json={"inputs": [5, 6, 7], "parameters": {"max_new_tokens": 2}},
                             timeout=60).status_code == 200:
                break
            time.sleep(1)
        results, started = [], threading.Event()

        def client(i):
            got, last, t_start = 0, b"", time.time()
            try:
                with requests.post(url + "/generate_stream", json={"inputs": list(range(5 + i, 60 + i)), "parameters": {
                        "max_new_tokens": 450, "ignore_eos": True}}, stream=True, timeout=120) as r:
                    for line in r.iter_lines():
                        if line.startswith(b"data:"):
                            got, last = got + 1, line
                            if got >= 3:
                                started.set()
                results.append((got, json.loads(last[5:]), time.time() - t_start))
            except Exception as e:  # noqa: BLE001
                results.append((got, {"exception": repr(e)}, time.time() - t_start))

        threads = [threading.Thread(target=client, args=(i,)) for i in range(3)]
        for t in threads:
            t.start()
        assert started.wait(60)
        os.killpg(decode.pid, signal.SIGKILL)
        killed = time.time()
        for t in threads:
            t.join(timeout=60)
        assert time.time() - killed < 30 and len(results) == 3, results
        for got, last, _ in results:
            assert 1 <= got < 450 and last.get("finished") and last.get("finish_reason") == "error", results
        r = requests.post(url + "/generate", json={"inputs": [1, 2, 3], "parameters": {"max_new_tokens": 3}}, timeout=30)
        assert r.status_code == 429 and "topology" in r.text
        decode2 = _spawn(common + ["--run_mode", "decode", "--port", str(pd2)] + flags, d / "decode2.log")
        procs.append(decode2)
        _wait_up(f"http://127.0.0.1:{pd2}", decode2, d / "decode2.log")
        t0, r = time.time(), None
        while time.time() - t0 < 60:
            r = requests.post(url + "/generate", json={"inputs": list(range(5, 40)), "parameters": {
                "max_new_tokens": 5, "ignore_eos": True}}, timeout=60)
            if r.status_code == 200:
                break
            time.sleep(1)
        assert r.status_code == 200 and r.json()["count_output_tokens"] == 5, r.text
        assert prefill.poll() is None and master.poll() is None
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
