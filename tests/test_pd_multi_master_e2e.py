"""Several pd_masters behind one config server: the masters register there and draw disjoint request-id ranges from
it, prefill / decode nodes find the masters in its list and keep a link to each; requests through either master give
the tokens of a single-process run, also when both masters drive the same pair of nodes at once."""
import json
import os
import signal
import subprocess
import threading
import time

import pytest
import requests

from test_pd_e2e import CFG, _free_port, _spawn, _wait_up


@pytest.mark.timeout(1500)
def test_two_masters_share_one_pair_of_nodes(tmp_path):
    from lightllm_b200.engine.llm import LLM

    d = tmp_path
    (d / "config.json").write_text(json.dumps(CFG))
    pc, m1, m2, pp, pdp = (_free_port() for _ in range(5))
    where = ["--config_server_host", "127.0.0.1", "--config_server_port", str(pc)]
    common = ["--model_dir", str(d), "--data_type", "fp32", "--max_total_token_num", "4096", "--running_max_req_size", "8",
              "--max_req_total_len", "256", "--tp", "1", "--host", "127.0.0.1", "--pd_kv_page_size", "16"] + where
    procs = []
    try:
        cs = _spawn(["--run_mode", "config_server"] + where, d / "config.log")
        procs.append(cs)
        _wait_up(f"http://127.0.0.1:{pc}", cs, d / "config.log")
        for k, port in enumerate((m1, m2)):
            procs.append(_spawn(["--run_mode", "pd_master", "--port", str(port), "--host", "127.0.0.1", "--model_dir", str(d),
                                 "--select_p_d_node_strategy", "round_robin"] + where, d / f"master{k}.log"))
        for k, port in enumerate((m1, m2)):
            _wait_up(f"http://127.0.0.1:{port}", procs[1 + k], d / f"master{k}.log")
        procs.append(_spawn(common + ["--run_mode", "prefill", "--port", str(pp)], d / "prefill.log"))
        procs.append(_spawn(common + ["--run_mode", "decode", "--port", str(pdp)], d / "decode.log"))
        _wait_up(f"http://127.0.0.1:{pp}", procs[3], d / "prefill.log")
        _wait_up(f"http://127.0.0.1:{pdp}", procs[4], d / "decode.log")
        llm = LLM(config=CFG, data_type="float32", max_total_token_num=2048, running_max_req_size=4,
                  max_req_total_len=256, batch_max_tokens=256)
        sp = {"max_new_tokens": 7, "ignore_eos": True}
        prompts = [list(range(7 + k, 50 + k)) for k in range(6)]
        want = [llm.generate([p], sp)[0]["token_ids"] for p in prompts]
        logs = lambda: "\n".join(f"--- {f.name}\n" + f.read_text()[-1200:] for f in sorted(d.glob("*.log")))  # noqa: E731
        for port in (m1, m2):          # the nodes link up with a master a few seconds after it has registered
            t0, r = time.time(), None
            while time.time() - t0 < 90:
                r = requests.post(f"http://127.0.0.1:{port}/generate", json={"inputs": prompts[0], "parameters": dict(
                    sp, return_details=True)}, timeout=120)
                if r.status_code == 200:
                    break
                time.sleep(2)
            assert r is not None and r.status_code == 200, (r.text if r is not None else "") + logs()
            assert [t["id"] for t in r.json()["tokens"]] == want[0], logs()
        # both masters at once on the same nodes: ids from disjoint ranges, every answer right
        got = {}

        def ask(i):
            port = (m1, m2)[i % 2]
            r = requests.post(f"http://127.0.0.1:{port}/generate", json={"inputs": prompts[i], "parameters": dict(
                sp, return_details=True)}, timeout=180)
            got[i] = [t["id"] for t in r.json()["tokens"]] if r.status_code == 200 else r.text

        threads = [threading.Thread(target=ask, args=(i,)) for i in range(6)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=200)
        assert [got.get(i) for i in range(6)] == want, logs()
        assert all(p.poll() is None for p in procs)
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
